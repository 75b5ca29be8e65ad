// Streaming decode GEMV for sm_100a: weights in any of the ten block formats (Q4_K, Q6_K, Q8_0, Q4_0, Q5_K, Q5_0,
// Q5_1, IQ4_NL, Q2_K, Q3_K), K a multiple of 256, 1..8 activation rows, up to 16 matrices per launch.
//
// Design (B200-first, not the reference's one-warp-per-row walk of src/hip/kernels/gemm.hpp:76):
//
//  * One persistent CTA per SM owns a contiguous range of output rows. A producer warp streams
//    that range through a ring of shared-memory stages with bulk-async copies (cp.async.bulk,
//    one copy per weight row so that rows land on a padded, bank-conflict-free stride) signalled
//    on mbarriers; 8 consumer warps never touch global memory for weights. The ring keeps
//    50-90 KB of HBM reads in flight per SM without spending registers on it.
//
//  * A CTA takes HALF an SM (320 threads, <= 113 KB of shared memory), so the CTA of the NEXT launch
//    in the stream becomes resident (programmatic dependent launch) while this one is still
//    streaming: it sets itself up and fills its ring with weights, which no kernel in flight
//    writes, and only then waits for this grid to complete before it reads activations. The gap
//    between two launches is then a CTA start, not a CTA start plus a pipeline fill.
//
//  * At 8 TB/s a B200 SM must retire ~40 four-bit weights per clock: unpacking each one to f32
//    and issuing an FMA for it does not fit the issue budget. So the dot products run on the
//    tensor cores as EXACT integer arithmetic: the quants are fed as s8 fragments straight from
//    the packed bytes (one AND per four nibbles) to mma.sync m16n8k32 / m16n8k16 (s8 x s8 -> s32),
//    16 output rows at a time, and the activation is held as three signed 8-bit limbs of a
//    23-bit fixed-point number (x ~ s * (l0*65536 + l1*256 + l2), |X| < 2^22), one limb per MMA column.
//    The products and sums are exact; the only rounding is the 23-bit quantisation of x
//    (relative to max|x|, i.e. f32-mantissa sized) and the final f32 scale arithmetic, so the
//    result sits well inside the 1e-4 * ||w_row|| * ||x|| bound. Sub-block scales are applied
//    to the s32 partial sums in integer arithmetic, block scales in f32.
//
//  * Because a dot product does not care about the order of its terms, each lane takes the
//    bytes that are cheapest to load and the activation limbs are laid out in the matching
//    order once per CTA.
//
// Every wait on an mbarrier is bounded; a wait that gives up raises the device status word
// and the CTA drains without touching memory it does not own.
#include <cuda.h>

#include <cfloat>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "krk_common.cuh"

namespace krk_cuda {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 64;   // warp 0: producer, warps 1..8: consumers, warp 9: epilogue
constexpr int kEpilogueWarp = kConsumerWarps + 1;
// Tiles whose partial sums may wait for the epilogue warp (fewer when more activation rows make a slot larger).
__host__ __device__ constexpr int red_slots(int ng) { return ng == 1 ? 4 : ng == 2 ? 2 : 1; }
constexpr int kMaxRedSlots = 4;
constexpr int kMaxStack = 4;      // 16-row tiles per stage at most
constexpr int kTileRows = 16;                     // the M of the MMA
constexpr int kMaxStages = 4;                    // measured: four stages in flight per CTA stream a large Q4_K matrix at 0.89 of the
                                                  // copy bandwidth, five (all that fit) at 0.86, three at 0.86
constexpr int kSmemLimit = 113 * 1024;           // two CTAs per SM (228 KB, 1 KB reserved per CTA)
constexpr int kSmemWhole = 227 * 1024;
constexpr int kPlanePad = 32;                     // bytes between limb planes beyond n_in: spreads the B-fragment loads over the banks
constexpr float kFixedOne = 4194303.0f;           // 2^22 - 1: every limb stays in s8 and X = rint(x / s) is one FMA against
                                                  // the bits of 1.5 * 2^23 (no conversion instruction)
constexpr long long kWaitCycles = 4000000000LL;   // ~2 s at boost clock, then give up

template <int WT> struct Fmt;
// tma: how a stage can arrive as ONE tiled tensor copy. 1: a unit is a whole number of 16-byte granules (Q4_K's
// 144 bytes): box {unit bytes, rows, units}, laid out [unit][row][unit bytes]. 2: eight units of a row are (Q6_K:
// 8 x 210 = 1680 bytes, as 210 64-bit elements): box {8 units, rows}, laid out [row][8 units], which is the
// layout of the per-row copies with a 1680-byte pitch. 0: per-row bulk copies only.
template <> struct Fmt<KRK_CUDA_Q4_K> { static constexpr int unit_values = 256, unit_bytes = 144, stride_mod = 32, tma = 1; };
template <> struct Fmt<KRK_CUDA_Q6_K> { static constexpr int unit_values = 256, unit_bytes = 210, stride_mod = 16, tma = 2; };
template <> struct Fmt<KRK_CUDA_Q8_0> { static constexpr int unit_values = 128, unit_bytes = 136, stride_mod = 16, tma = 0; };
// Q5_K: Q4_K's header and nibbles with 32 bytes of fifth bits between them (src/quant.cpp:462-489).
template <> struct Fmt<KRK_CUDA_Q5_K> { static constexpr int unit_values = 256, unit_bytes = 176, stride_mod = 32, tma = 1; };
// Q4_0: eight 18-byte blocks are 144 bytes, the size of a Q4_K unit, so the stages are laid out the same way.
template <> struct Fmt<KRK_CUDA_Q4_0> { static constexpr int unit_values = 256, unit_bytes = 144, stride_mod = 16, tma = 1; };
// Q5_0: eight 22-byte blocks are 176 bytes, the size of a Q5_K unit (rows of a fragment load 44 words apart: no
// bank is met twice). Q5_1: eight 24-byte blocks are 192 bytes, a pitch that would put rows g and g + 2 on the
// same banks, so its stages arrive as per-row copies with a padded pitch.
template <> struct Fmt<KRK_CUDA_Q5_0> { static constexpr int unit_values = 256, unit_bytes = 176, stride_mod = 16, tma = 1; };
// Q2_K (84 bytes) and Q3_K (110 bytes): per-row copies; rows that are not 16-byte multiples go the ragged way.
template <> struct Fmt<KRK_CUDA_Q2_K> { static constexpr int unit_values = 256, unit_bytes = 84, stride_mod = 16, tma = 0; };
template <> struct Fmt<KRK_CUDA_Q3_K> { static constexpr int unit_values = 256, unit_bytes = 110, stride_mod = 16, tma = 0; };
// IQ4_NL: Q4_0's block with grid indices in place of quants.
template <> struct Fmt<KRK_CUDA_IQ4_NL> { static constexpr int unit_values = 256, unit_bytes = 144, stride_mod = 16, tma = 1; };
template <> struct Fmt<KRK_CUDA_Q5_1> { static constexpr int unit_values = 256, unit_bytes = 192, stride_mod = 16, tma = 0; };

struct StreamParams {
    GemvMat mat[KRK_CUDA_MAX_GROUP];
    int gran_begin[KRK_CUDA_MAX_GROUP + 1];   // first row granule of each entry
    int n_entries;        // matrices, or gate/up pairs when silu_pair
    int step;             // matrices per entry (2 for gate/up pairs)
    int rows;             // activation rows
    int accumulate;
    int n_in;
    int units;            // n_in / unit_values
    int row_bytes;
    int gran;             // rows per granule: 1, or 8 when rows are not 16-byte multiples
    int whole_tiles;      // 1: a stage is one contiguous copy of whole rows (unaligned row size)
    int ragged;           // 1: rows are not 16-byte multiples and too long for whole tiles: every row of a stage is
                          // copied from the 16-byte boundary below its first byte, and its bytes sit that far
                          // (0..15 bytes, a multiple of 2) into the row's slot
    int tps;              // 16-row tiles stacked in one stage (> 1 when a row has so few K units that one
                          // tile would leave most consumer warps idle: warp w takes unit w % units of
                          // sub-tile w / units)
    int row_stride;       // bytes between rows inside a stage
    int unit_stride;      // bytes between the K units of one row group inside a stage
    int use_tma;          // 1: a stage arrives as one tiled tensor copy, laid out [unit][row][unit_bytes]; 2: [row][units]
    int tma_unit_div;     // the copy's third coordinate is the stage's first unit / this
    int box_bytes;        // bytes one tensor copy signals (the whole box, also where the matrix clips it)
    int tune;             // experiment bits: 1 = weights are not prefetched before the dependency wait; 2 = the dependent
                          // launch is released after this grid's own dependency wait instead of at its start
    int stage_bytes;
    int n_stages;
    int total_gran;
    int gran_q, gran_r;   // total_gran = grid * gran_q + gran_r
    const StreamTable *dev_table;   // when set, matrices and granule prefix come from device memory
    // Table launches with tensor copies: every matrix of the table lies inside one of two stacked banks (the gate
    // and the up bank of an expert set), each described by ONE tensor map (wmap[0], wmap[1]) over all of its
    // rows; a matrix is then a row offset into its bank.
    const uint8_t *bank_base[2];
    // Fused all-gather (single-matrix launches of a row shard): y goes to slot `peer_offset` of the full
    // output row in every peer's memory (this GPU's own buffer included), then the peers are told.
    float *peer_y[KRK_CUDA_MAX_PEERS];
    int *peer_flag[KRK_CUDA_MAX_PEERS];   // peer_flag[q][my_rank] <- epoch once every CTA here has stored
    int n_peers, my_rank, epoch, wait_peers;
    long long peer_row_stride, peer_offset;
    int *status;
    // per matrix: the weights as a 3-d tensor {unit_bytes, n_out rows, units per row}; box = {unit_bytes,
    // rows of a stage, units of a stage}
    CUtensorMap wmap[KRK_CUDA_MAX_GROUP];
};


// ---- PTX wrappers ----------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// One tiled tensor copy global -> shared (no multicast): box origin (0, row, unit).
__device__ __forceinline__ void tma_box(uint32_t dst, const CUtensorMap *map, int row, int unit, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(0), "r"(row), "r"(unit), "r"(bar) : "memory");
}
// c = A x B with a zero accumulator input (the sub-block scale is applied to c afterwards).
__device__ __forceinline__ void mma_s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// The same with unsigned A bytes (raw nibble pairs q_lo + 16 q_hi, or masked nibbles).
__device__ __forceinline__ void mma_u8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// k16 with the accumulator preset to the bits of 1.5 * 2^23: for |sum| < 2^22 the s32 result read as a
// float is exactly 12582912 + sum, so the conversion to float costs one subtraction instead of an I2F.
constexpr float kMagic = 12582912.0f;
__device__ __forceinline__ void mma_s8_k16_biased(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    int r[4];
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0x4B400000));
#pragma unroll
    for (int i = 0; i < 4; i++) c[i] = __int_as_float(r[i]) - kMagic;
}
// the k16 form adding onto an accumulator that already holds the biased sum of an earlier MMA
__device__ __forceinline__ void mma_s8_k16_chain(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mma_u8_k16_chain(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ void mma_u8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
__device__ __forceinline__ void mma_s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// x << log2(M), issued as a multiply-add: the units below are bound by the integer ALU pipe (shifts, logic ops,
// byte permutes) while the multiply-add pipe idles, so the left shifts of the operand assembly go there. The
// compiler turns a plain `x * M` back into a shift.
template <uint32_t M>
__device__ __forceinline__ uint32_t shl_mad(uint32_t x) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, 0;" : "=r"(r) : "r"(x), "n"(M));
    return r;
}
__device__ __forceinline__ uint32_t shl_mad_n(uint32_t x, int k) {   // k is a constant once the caller's loops are unrolled
    switch (k) {
    case 1: return shl_mad<2u>(x);
    case 2: return shl_mad<4u>(x);
    case 3: return shl_mad<8u>(x);
    case 4: return shl_mad<16u>(x);
    default: return x << k;
    }
}
__device__ __forceinline__ int sext_byte(uint32_t w, int i) {
    int r;
    asm("bfe.s32 %0, %1, %2, 8;" : "=r"(r) : "r"(w), "r"(8 * i));
    return r;
}
__device__ __forceinline__ float half_lo(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu))); }
__device__ __forceinline__ float half_hi(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }

// Bounded wait on an mbarrier phase. Once any wait in the CTA has given up, every later wait
// returns at once, so the CTA runs to its end (on stale data, inside its own buffers) instead
// of hanging.
__device__ __noinline__ void wait_phase_slow(uint32_t bar, uint32_t parity, volatile int *gave_up, int *status) {
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 32; i++) {
            if (mbar_try_wait(bar, parity)) return;
            __nanosleep(20);   // leave the issue slots to the warps that have work
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
    wait_phase_slow(bar, parity, gave_up, status);
}

// ---- shared-memory map ---------------------------------------------------------------------------

template <int NG>
struct Smem {
    unsigned long long full[kMaxStages];     // weights of a stage have landed
    unsigned long long empty[kMaxStages];    // every consumer warp is done with the stage
    unsigned long long red_full[kMaxRedSlots];  // every consumer warp has written its partial sums of a tile
    unsigned long long red_empty[kMaxRedSlots]; // the epilogue warp has consumed them
    int gave_up;
    int pad[3];
    float gate[kMaxStack][NG][32];   // epilogue warp: the gate tile(s) of a gate/up pair, until the up tile arrives
    // per consumer warp, column group and row pair (g, g+8): {row g x even activation row, g x odd, g+8 x even, g+8 x odd}
    float4 red[red_slots(NG)][kConsumerWarps][NG][8];
};

__host__ __device__ constexpr int align_up(int v, int a) { return (v + a - 1) / a * a; }

__host__ __device__ inline int plane_stride(int n_in) { return n_in + kPlanePad; }
template <int WT>
__host__ __device__ inline int plane_bytes(int n_in, int rows) { return align_up(rows * 3 * plane_stride(n_in), 128); }
// Sums of the quantised activation over the stretch of K that shares one minimum or offset: 32 values (2^5) for
// Q4_K, Q5_K, Q4_0 and Q5_1, 16 for Q2_K.
template <int WT>
constexpr int kSumShift = WT == KRK_CUDA_Q2_K ? 4 : 5;
template <int WT>
__host__ __device__ inline int chunk_sum_bytes(int n_in, int rows) {   // [row][4 limbs][n_in >> kSumShift] s8
    return (WT == KRK_CUDA_Q4_K || WT == KRK_CUDA_Q5_K || WT == KRK_CUDA_Q4_0 || WT == KRK_CUDA_Q5_1 || WT == KRK_CUDA_Q2_K)
               ? align_up(rows * (n_in >> kSumShift<WT>) * 4, 128) : 0;   // Q4_0, Q5_1: [row][n_in / 32] f32
}

// ---- the walk over this CTA's stages: identical in the producer and in the consumers -------------

struct StageInfo {
    int mat;        // matrix index
    int which;      // 0, or 1 for the `up` half of a gate/up pair
    int row0;       // first output row of the tile
    int n_rows;     // valid rows in the stage (1..16 * tps)
    int unit0;      // first K unit of this stage
    int n_units;    // units in this stage (1..16)
    int last;       // last stage of the tile
    int slot;       // ring slot of this stage
    int phase;      // parity of the slot's current use
};

// Where the list of matrices lives: the kernel parameters (host-built launches) or a table in
// device memory written by an earlier kernel (the routed-expert launches, whose matrices depend on
// expert ids that never leave the device).
struct TableView {
    const GemvMat *mat;
    const int *gran_begin;
    int n_entries;
    int gran_q, gran_r;
};

__device__ __forceinline__ TableView table_view(const StreamParams &p) {
    TableView tv;
    if (p.dev_table) {
        tv.mat = p.dev_table->mat;
        tv.gran_begin = p.dev_table->gran_begin;
        tv.n_entries = p.dev_table->n_entries;
        const int total = p.dev_table->total_gran;
        tv.gran_q = total / (int)gridDim.x;
        tv.gran_r = total % (int)gridDim.x;
    } else {
        tv.mat = p.mat;
        tv.gran_begin = p.gran_begin;
        tv.n_entries = p.n_entries;
        tv.gran_q = p.gran_q;
        tv.gran_r = p.gran_r;
    }
    return tv;
}

template <class SegmentFn, class StageFn>
__device__ __forceinline__ void walk(const StreamParams &p, const TableView &tv, int tps, SegmentFn &&on_segment, StageFn &&on_stage) {
    // balanced split of the granules over the CTAs: the first gran_r CTAs take one more
    const int c = (int)blockIdx.x;
    const int g0 = c * tv.gran_q + min(c, tv.gran_r);
    const int g1 = g0 + tv.gran_q + (c < tv.gran_r ? 1 : 0);
    const int ku_max = p.whole_tiles ? p.units : kConsumerWarps;
    int slot = 0, phase = 0;
    for (int e = 0; e < tv.n_entries; e++) {
        const int lo = max(g0, tv.gran_begin[e]), hi = min(g1, tv.gran_begin[e + 1]);
        if (lo >= hi) continue;
        const int n_out = (int)tv.mat[e * p.step].n_out;
        const int r0 = (lo - tv.gran_begin[e]) * p.gran;
        const int r1 = min(n_out, (hi - tv.gran_begin[e]) * p.gran);
        on_segment(e * p.step);
        const int stage_rows = kTileRows * tps;
        for (int tr = r0; tr < r1; tr += stage_rows) {
            for (int which = 0; which < p.step; which++) {
                for (int u0 = 0; u0 < p.units; u0 += ku_max) {
                    StageInfo s;
                    s.mat = e * p.step + which;
                    s.which = which;
                    s.row0 = tr;
                    s.n_rows = min(stage_rows, r1 - tr);
                    s.unit0 = u0;
                    s.n_units = min(ku_max, p.units - u0);
                    s.last = u0 + ku_max >= p.units;
                    s.slot = slot;
                    s.phase = phase;
                    if (++slot == p.n_stages) {
                        slot = 0;
                        phase ^= 1;
                    }
                    on_stage(s);
                }
            }
        }
    }
}

// ---- activation preparation -------------------------------------------------------------------------
// Consumer warp w only ever multiplies K units w, w+16, ... so it prepares exactly those slices
// of x itself: no other warp reads them and no CTA-wide barrier is involved. Per activation row:
// s = max|x| / (127 * 2^16) over the warp's slices, X = rint(x / s) as three balanced s8 limbs
// written as byte planes [row][limb][k] in the order the B fragments are read, and (Q4_K) the
// integer sum of X over every 32-value chunk as four balanced s8 limbs [row][limb][chunk] for
// the `min` term. s is returned (NaN when a slice holds a non-finite activation, so the output
// becomes NaN as it would in f32) and multiplies the warp's partial sums at the end of each tile.

__device__ __forceinline__ int sext8(int v) { return (v << 24) >> 24; }

// Balanced signed-byte limbs of a fixed-point value: adding 128 at every byte position turns the limbs
// l in [-128, 127] into the bytes l + 128 of an unsigned number (carries do the balancing), and flipping
// bit 7 of every byte turns l + 128 back into l as a two's complement byte.
__device__ __forceinline__ uint32_t limbs3(int X) { return ((uint32_t)X + 0x00808080u) ^ 0x00808080u; }   // |X| < 2^23
__device__ __forceinline__ uint32_t limbs4(int X) { return ((uint32_t)X + 0x80808080u) ^ 0x80808080u; }

template <int WT>
__device__ __forceinline__ void quantize_slice(const float (&f)[Fmt<WT>::unit_values / 32], float inv, int k0, int8_t *p0,
                                               int8_t *p1, int8_t *p2, int8_t *sums, int n_chunks, int lane) {
    constexpr int PER = Fmt<WT>::unit_values / 32;
    int total = 0;
#pragma unroll
    for (int j4 = 0; j4 < PER; j4 += 4) {
        uint32_t z[4];   // byte 0: limb 2 (weight 1), byte 1: limb 1 (256), byte 2: limb 0 (65536)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int X = __float_as_int(fmaf(f[j4 + j], inv, kMagic)) - 0x4B400000;   // |x * inv| < 2^22
            total += X;
            z[j] = limbs3(X);
        }
        const uint32_t lo01 = __byte_perm(z[0], z[1], 0x5140), lo23 = __byte_perm(z[2], z[3], 0x5140);   // l2a l2b l1a l1b
        const uint32_t w2 = __byte_perm(lo01, lo23, 0x5410), w1 = __byte_perm(lo01, lo23, 0x7632);
        const uint32_t w0 = __byte_perm(__byte_perm(z[0], z[1], 0x0062), __byte_perm(z[2], z[3], 0x0062), 0x5410);
        const int i = k0 + j4;
        if (WT == KRK_CUDA_Q8_0 && ((i >> 5) & 1) == 0) {
            // Even blocks start 2 bytes off a word boundary, so their lanes take the quants in the
            // order [0,1,30,31, 2..29]; the limbs follow: pair (e, e+1) lands at position pos(e).
            const int e = i & 31, base = i & ~31;
            const int ka = e < 2 ? e : (e >= 30 ? e - 28 : e + 2);
            const int e2 = e + 2;
            const int kb = e2 < 2 ? e2 : (e2 >= 30 ? e2 - 28 : e2 + 2);
            *reinterpret_cast<uint16_t *>(p0 + base + ka) = (uint16_t)(w0 & 0xFFFF);
            *reinterpret_cast<uint16_t *>(p0 + base + kb) = (uint16_t)(w0 >> 16);
            *reinterpret_cast<uint16_t *>(p1 + base + ka) = (uint16_t)(w1 & 0xFFFF);
            *reinterpret_cast<uint16_t *>(p1 + base + kb) = (uint16_t)(w1 >> 16);
            *reinterpret_cast<uint16_t *>(p2 + base + ka) = (uint16_t)(w2 & 0xFFFF);
            *reinterpret_cast<uint16_t *>(p2 + base + kb) = (uint16_t)(w2 >> 16);
        } else if (WT == KRK_CUDA_Q5_0 && ((i >> 5) & 1) == 0) {
            // As Q4_0, [16 of the low half][16 of the high half], but the quants of an even block start 6 bytes
            // into it: its lanes take them rotated by two, [14,15, 0..13], so that lane t holds values 4t-2..4t+1
            // of a half and their fifth bits are four neighbours of the rotated mask.
            const int e = i & 15, base = (i & ~31) + (i & 16);
            const int ka = (e + 2) & 15, kb = (e + 4) & 15;
            *reinterpret_cast<uint16_t *>(p0 + base + ka) = (uint16_t)(w0 & 0xFFFF);
            *reinterpret_cast<uint16_t *>(p0 + base + kb) = (uint16_t)(w0 >> 16);
            *reinterpret_cast<uint16_t *>(p1 + base + ka) = (uint16_t)(w1 & 0xFFFF);
            *reinterpret_cast<uint16_t *>(p1 + base + kb) = (uint16_t)(w1 >> 16);
            *reinterpret_cast<uint16_t *>(p2 + base + ka) = (uint16_t)(w2 & 0xFFFF);
            *reinterpret_cast<uint16_t *>(p2 + base + kb) = (uint16_t)(w2 >> 16);
        } else if (WT == KRK_CUDA_Q4_0 || WT == KRK_CUDA_IQ4_NL) {
            // A block's 16 quant bytes hold value j in their low and value 16 + j in their high nibbles, so the
            // limbs of a block lie as [16 of the low half][16 of the high half], each in the order the lanes take
            // the quant bytes: as they are in odd blocks; [0,1,14,15, 2..13] in even blocks, whose quants start
            // 2 bytes off a word boundary (pairs stay together, as for Q8_0).
            const int e = i & 15, base = (i & ~31) + (i & 16);
            if (((i >> 5) & 1) == 0) {
                const int e2 = e + 2;
                const int ka = e < 2 ? e : (e >= 14 ? e - 12 : e + 2);
                const int kb = e2 < 2 ? e2 : (e2 >= 14 ? e2 - 12 : e2 + 2);
                *reinterpret_cast<uint16_t *>(p0 + base + ka) = (uint16_t)(w0 & 0xFFFF);
                *reinterpret_cast<uint16_t *>(p0 + base + kb) = (uint16_t)(w0 >> 16);
                *reinterpret_cast<uint16_t *>(p1 + base + ka) = (uint16_t)(w1 & 0xFFFF);
                *reinterpret_cast<uint16_t *>(p1 + base + kb) = (uint16_t)(w1 >> 16);
                *reinterpret_cast<uint16_t *>(p2 + base + ka) = (uint16_t)(w2 & 0xFFFF);
                *reinterpret_cast<uint16_t *>(p2 + base + kb) = (uint16_t)(w2 >> 16);
            } else {
                *reinterpret_cast<uint32_t *>(p0 + base + e) = w0;
                *reinterpret_cast<uint32_t *>(p1 + base + e) = w1;
                *reinterpret_cast<uint32_t *>(p2 + base + e) = w2;
            }
        } else {
            *reinterpret_cast<uint32_t *>(p0 + i) = w0;
            *reinterpret_cast<uint32_t *>(p1 + i) = w1;
            *reinterpret_cast<uint32_t *>(p2 + i) = w2;
        }
    }
    if (WT == KRK_CUDA_Q4_0 || WT == KRK_CUDA_Q5_1) {
        // the sum of X over each 32-value block, as a float: the -8 of every quant leaves -8 * d * sum per block
        // (Q5_1: the block's offset m enters as m * sum)
        total += __shfl_xor_sync(0xFFFFFFFFu, total, 1);
        total += __shfl_xor_sync(0xFFFFFFFFu, total, 2);
        if ((lane & 3) == 0) reinterpret_cast<float *>(sums)[k0 >> 5] = (float)total;   // |sum| < 2^28
    }
    if (WT == KRK_CUDA_Q4_K || WT == KRK_CUDA_Q5_K || WT == KRK_CUDA_Q2_K) {
        // a 32-value chunk is held by 4 consecutive lanes (Q2_K: a 16-value group by 2); |sum| <= 32 * 2^22
        constexpr int kLanes = WT == KRK_CUDA_Q2_K ? 2 : 4;
        total += __shfl_xor_sync(0xFFFFFFFFu, total, 1);
        if (kLanes == 4) total += __shfl_xor_sync(0xFFFFFFFFu, total, 2);
        if ((lane & (kLanes - 1)) == 0) {
            const int c = k0 >> kSumShift<WT>;
            const uint32_t z = limbs4(total);   // byte 0: limb 3 (weight 1) ... byte 3: limb 0 (2^24)
            sums[c] = (int8_t)(z >> 24);
            sums[n_chunks + c] = (int8_t)(z >> 16);
            sums[2 * n_chunks + c] = (int8_t)(z >> 8);
            sums[3 * n_chunks + c] = (int8_t)z;
        }
    }
}

// (the running maximum is kept on the bit patterns of |x|: they order like the values, and anything above the
// largest finite pattern is an infinity or a NaN)
template <int WT>
__device__ __forceinline__ void load_slice(const float *__restrict__ x, int k0, float (&f)[Fmt<WT>::unit_values / 32],
                                           uint32_t &mxb) {
    constexpr int PER = Fmt<WT>::unit_values / 32;
#pragma unroll
    for (int j = 0; j < PER; j += 4) {
        const float4 v = *reinterpret_cast<const float4 *>(x + k0 + j);
        f[j] = v.x; f[j + 1] = v.y; f[j + 2] = v.z; f[j + 3] = v.w;
    }
#pragma unroll
    for (int j = 0; j < PER; j++) mxb = max(mxb, __float_as_uint(f[j]) & 0x7FFFFFFFu);
}

// All slices this warp will read of one activation row; returns the row's scale for this warp.
template <int WT>
__device__ __forceinline__ float prepare_x_row(const float *__restrict__ xr, const StreamParams &p, int8_t *p0, int8_t *sums,
                                               int wid, int lane) {
    constexpr int UV = Fmt<WT>::unit_values, PER = UV / 32, kHeld = 2;
    const int n_chunks = p.n_in >> kSumShift<WT>, ps = plane_stride(p.n_in);
    // the first two slices stay in registers between the max and the quantisation (K <= 4096 for
    // 256-value units); any further ones are read twice
    float held[kHeld][PER];
    uint32_t mxb = 0u;
#pragma unroll
    for (int j = 0; j < kHeld; j++) {
        const int u = wid + j * kConsumerWarps;
        if (u < p.units) load_slice<WT>(xr, u * UV + lane * PER, held[j], mxb);
    }
    for (int u = wid + kHeld * kConsumerWarps; u < p.units; u += kConsumerWarps) {
        float f[PER];
        load_slice<WT>(xr, u * UV + lane * PER, f, mxb);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mxb = max(mxb, __shfl_xor_sync(0xFFFFFFFFu, mxb, o));
    const bool bad = mxb > 0x7F7FFFFFu;
    const float mx = __uint_as_float(mxb);
    const float inv = (mx > 0.0f && !bad) ? __fdiv_rn(kFixedOne, mx) : 0.0f;
#pragma unroll
    for (int j = 0; j < kHeld; j++) {
        const int u = wid + j * kConsumerWarps;
        if (u < p.units)
            quantize_slice<WT>(held[j], inv, u * UV + lane * PER, p0, p0 + ps, p0 + 2 * ps, sums, n_chunks, lane);
    }
    for (int u = wid + kHeld * kConsumerWarps; u < p.units; u += kConsumerWarps) {
        float f[PER];
        uint32_t m2 = 0u;
        load_slice<WT>(xr, u * UV + lane * PER, f, m2);
        quantize_slice<WT>(f, inv, u * UV + lane * PER, p0, p0 + ps, p0 + 2 * ps, sums, n_chunks, lane);
    }
    return bad ? __int_as_float(0x7FC00000) : __fdiv_rn(mx, kFixedOne);
}

// ---- per-format unit kernels -------------------------------------------------------------------------
// A unit is 256 values (128 for Q8_0) of 16 weight rows: lane (g, t) = (lane/4, lane%4) holds the
// A fragments of rows g and g+8, column g of the B fragment (limb g%3 of activation row g/3 of
// the column group), and accumulator columns 2t, 2t+1.

// Column groups that go through the MMAs. One or two groups carry two activation rows each in columns 0..5. The
// form for five to eight rows has four groups of outputs but multiplies only three: rows 0..5 sit in columns 0..5
// of groups 0..2 and rows 6 and 7 in the spare columns 6 and 7, limb mg of the row in group mg, so that 24 columns
// carry 8 rows x 3 limbs with none to spare.
template <int NG>
constexpr int kMmaGroups = NG == 4 ? 3 : NG;

template <int NG>
struct Accum {
    float f[NG][4];   // [group][(row g | g+8) x (col 2t | 2t+1)], already times the block scale d
    float m[NG][4];   // Q4_K: the same for dmin * sum(min_c * sum_X_c), columns = 4 limbs x 2 activation rows
};

template <int NG>
__device__ __forceinline__ void accum_zero(Accum<NG> &a) {
#pragma unroll
    for (int i = 0; i < NG; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) a.f[i][j] = 0.0f;
#pragma unroll
    for (int i = 0; i < NG; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) a.m[i][j] = 0.0f;
}

// Byte planes this lane reads its B fragments from, one per column group. A lane whose column
// carries no limb (columns 6, 7, or an activation row past `rows`) reads some valid plane: its
// accumulator columns are never looked at, so what it multiplies does not matter.
template <int NG>
__device__ __forceinline__ void lane_planes(const int8_t *planes, const int8_t *chunk_sum, int n_in, int n_sums, int rows, int g,
                                            const int8_t *(&bp)[NG], const int8_t *(&sp)[NG]) {
#pragma unroll
    for (int mg = 0; mg < NG; mg++) {
        int r = 2 * mg + (g % 6) / 3, limb = g % 3;
        if (NG == 4 && g >= 6) {   // the spare columns: limb mg of activation row 6 or 7 (group 3 multiplies nothing)
            r = g;
            limb = mg % 3;
        }
        r = min(r, rows - 1);
        bp[mg] = planes + (size_t)(r * 3 + limb) * plane_stride(n_in);
        // chunk sums: column c = limb c%4 of activation row c/4 of the group
        const int rs = min(2 * mg + g / 4, rows - 1);
        sp[mg] = chunk_sum + (size_t)(rs * 4 + g % 4) * n_sums;
    }
}

// FIFTH: the Q5_K super-block: 32 bytes after the header whose bit c is the fifth quant bit of chunk c's value at the
// same position; the nibbles follow them.
template <int NG, bool FIFTH>
__device__ __forceinline__ void unit_q4_k(const uint8_t *rowA, const uint8_t *rowB, int kbase, const int8_t *const (&bp)[NG],
                                          const int8_t *const (&sp)[NG], int t, Accum<NG> &acc) {
    constexpr int kQs = FIFTH ? 48 : 16;
    const uint4 hA = *reinterpret_cast<const uint4 *>(rowA);
    const uint4 hB = *reinterpret_cast<const uint4 *>(rowB);
    uint2 fa = make_uint2(0u, 0u), fb = make_uint2(0u, 0u);
    if (FIFTH) {
        fa = *reinterpret_cast<const uint2 *>(rowA + 16 + 8 * t);
        fb = *reinterpret_cast<const uint2 *>(rowB + 16 + 8 * t);
    }
    // 6-bit scales and mins of the 8 chunks, four per word (src/quant.cpp:427-435 done bytewise)
    const uint32_t scA[2] = {hA.y & 0x3F3F3F3Fu, (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u)};
    const uint32_t scB[2] = {hB.y & 0x3F3F3F3Fu, (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u)};
    const uint32_t mnA[2] = {hA.z & 0x3F3F3F3Fu, ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u)};
    const uint32_t mnB[2] = {hB.z & 0x3F3F3F3Fu, ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u)};
    int I[NG][4];
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++)
#pragma unroll
        for (int j = 0; j < 4; j++) I[mg][j] = 0;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const uint2 qa = *reinterpret_cast<const uint2 *>(rowA + kQs + 32 * p + 8 * t);
        const uint2 qb = *reinterpret_cast<const uint2 *>(rowB + kQs + 32 * p + 8 * t);
#pragma unroll
        for (int nib = 0; nib < 2; nib++) {
            const int c = 2 * p + nib;
            uint32_t a0 = (qa.x >> (4 * nib)) & 0x0F0F0F0Fu, a1 = (qb.x >> (4 * nib)) & 0x0F0F0F0Fu;
            uint32_t a2 = (qa.y >> (4 * nib)) & 0x0F0F0F0Fu, a3 = (qb.y >> (4 * nib)) & 0x0F0F0F0Fu;
            if (FIFTH) {   // bit c of the mask bytes becomes bit 4 of the quants (0..31: still positive as s8)
                a0 |= (c < 4 ? shl_mad_n(fa.x, 4 - c) : fa.x >> (c - 4)) & 0x10101010u;
                a1 |= (c < 4 ? shl_mad_n(fb.x, 4 - c) : fb.x >> (c - 4)) & 0x10101010u;
                a2 |= (c < 4 ? shl_mad_n(fa.y, 4 - c) : fa.y >> (c - 4)) & 0x10101010u;
                a3 |= (c < 4 ? shl_mad_n(fb.y, 4 - c) : fb.y >> (c - 4)) & 0x10101010u;
            }
            const int sa = (scA[c >> 2] >> (8 * (c & 3))) & 0xFF, sb = (scB[c >> 2] >> (8 * (c & 3))) & 0xFF;
#pragma unroll
            for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
                const uint2 b = *reinterpret_cast<const uint2 *>(bp[mg] + kbase + 32 * c + 8 * t);
                int cc[4];
                mma_s8_k32(cc, a0, a1, a2, a3, b.x, b.y);
                I[mg][0] += sa * cc[0];
                I[mg][1] += sa * cc[1];
                I[mg][2] += sb * cc[2];
                I[mg][3] += sb * cc[3];
            }
        }
    }
    const float dA = half_lo(hA.x), dB = half_lo(hB.x);
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
        acc.f[mg][0] = fmaf(dA, (float)I[mg][0], acc.f[mg][0]);
        acc.f[mg][1] = fmaf(dA, (float)I[mg][1], acc.f[mg][1]);
        acc.f[mg][2] = fmaf(dB, (float)I[mg][2], acc.f[mg][2]);
        acc.f[mg][3] = fmaf(dB, (float)I[mg][3], acc.f[mg][3]);
    }
    // min term, also exact: one k16 MMA of the 8 mins of the super-block (k slots 0..7) against the
    // per-chunk sums of X, held as 4 limbs x 2 activation rows in the 8 columns
    const float nA = half_hi(hA.x), nB = half_hi(hB.x);
    const uint32_t a0 = t < 2 ? mnA[t & 1] : 0u, a1 = t < 2 ? mnB[t & 1] : 0u;
#pragma unroll
    for (int mg = 0; mg < NG; mg++) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(sp[mg] + (kbase >> 5) + 4 * (t & 1));
        int cc[4];
        mma_s8_k16(cc, a0, a1, b0);
        acc.m[mg][0] = fmaf(nA, (float)cc[0], acc.m[mg][0]);
        acc.m[mg][1] = fmaf(nA, (float)cc[1], acc.m[mg][1]);
        acc.m[mg][2] = fmaf(nB, (float)cc[2], acc.m[mg][2]);
        acc.m[mg][3] = fmaf(nB, (float)cc[3], acc.m[mg][3]);
    }
}

// Q4_K with ONE activation row: both nibbles of a byte go through the tensor core unshifted.
// The 32 bytes of a group hold chunk 2p in their low nibbles and chunk 2p+1 in their high ones.
// Column 2j of the B fragment carries limb j of x over chunk 2p, column 2j+1 limb j over chunk
// 2p+1. Two MMAs per group: L = (bytes & 0x0F) x B and R = (raw bytes) x B. Then, per limb,
//   low chunk  = L[even column],     high chunk = (R[odd column] - L[odd column]) / 16,
// because raw = q_lo + 16 q_hi. One AND per four bytes replaces the AND, shift, AND of the
// two-MMA-per-chunk form; lane t keeps limb t of rows g and g+8 (t = 3 multiplies nothing).
struct AccumSingle {
    float f[2];   // rows g, g+8: limb t of d * sum over sub-blocks, times 16
    float m[4];   // the min term as in Accum::m of one column group
};
// The B fragments of a unit (x limbs, chunk sums) are the same for every row tile: a warp that always works
// on the same K units keeps them in registers (BFrag) instead of reading them from shared memory per tile.
struct BFrag {
    uint2 b[4];     // per group of two chunks
    uint32_t m;     // chunk sums for the min term
};
__device__ __forceinline__ BFrag load_bfrag(const int8_t *bq, const int8_t *sq, int t) {
    BFrag f;
#pragma unroll
    for (int p = 0; p < 4; p++) f.b[p] = *reinterpret_cast<const uint2 *>(bq + 64 * p + 8 * t);
    f.m = *reinterpret_cast<const uint32_t *>(sq + 4 * (t & 1));
    return f;
}
__device__ __forceinline__ void unit_q4_k_single(const uint8_t *rowA, const uint8_t *rowB, const BFrag &bf, int t,
                                                 AccumSingle &acc) {
    const uint4 hA = *reinterpret_cast<const uint4 *>(rowA);
    const uint4 hB = *reinterpret_cast<const uint4 *>(rowB);
    const uint32_t scA[2] = {hA.y & 0x3F3F3F3Fu, (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u)};
    const uint32_t scB[2] = {hB.y & 0x3F3F3F3Fu, (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u)};
    const uint32_t mnA[2] = {hA.z & 0x3F3F3F3Fu, ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u)};
    const uint32_t mnB[2] = {hB.z & 0x3F3F3F3Fu, ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u)};
    int loA = 0, hrA = 0, hlA = 0, loB = 0, hrB = 0, hlB = 0;
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const uint2 qa = *reinterpret_cast<const uint2 *>(rowA + 16 + 32 * p + 8 * t);
        const uint2 qb = *reinterpret_cast<const uint2 *>(rowB + 16 + 32 * p + 8 * t);
        const uint2 b = bf.b[p];
        int cl[4], cr[4];
        mma_u8_k32(cl, qa.x & 0x0F0F0F0Fu, qb.x & 0x0F0F0F0Fu, qa.y & 0x0F0F0F0Fu, qb.y & 0x0F0F0F0Fu, b.x, b.y);
        mma_u8_k32(cr, qa.x, qb.x, qa.y, qb.y, b.x, b.y);
        const int c0 = 2 * p, c1 = 2 * p + 1;
        const int sA0 = (scA[c0 >> 2] >> (8 * (c0 & 3))) & 0xFF, sA1 = (scA[c1 >> 2] >> (8 * (c1 & 3))) & 0xFF;
        const int sB0 = (scB[c0 >> 2] >> (8 * (c0 & 3))) & 0xFF, sB1 = (scB[c1 >> 2] >> (8 * (c1 & 3))) & 0xFF;
        loA += sA0 * cl[0];
        hrA += sA1 * cr[1];
        hlA += sA1 * cl[1];
        loB += sB0 * cl[2];
        hrB += sB1 * cr[3];
        hlB += sB1 * cl[3];
    }
    // |16 lo + hr - hl| < 2^29: 4 groups x 63 x 32 x (16 * 15 + 255 + 15) x 128
    const float dA = half_lo(hA.x), dB = half_lo(hB.x);
    acc.f[0] = fmaf(dA, (float)(16 * loA + hrA - hlA), acc.f[0]);
    acc.f[1] = fmaf(dB, (float)(16 * loB + hrB - hlB), acc.f[1]);
    const float nA = half_hi(hA.x), nB = half_hi(hB.x);
    const uint32_t a0 = t < 2 ? mnA[t & 1] : 0u, a1 = t < 2 ? mnB[t & 1] : 0u;
    float cm[4];
    mma_s8_k16_biased(cm, a0, a1, bf.m);   // |sum| <= 8 x 63 x 128 < 2^22
    acc.m[0] = fmaf(nA, cm[0], acc.m[0]);
    acc.m[1] = fmaf(nA, cm[1], acc.m[1]);
    acc.m[2] = fmaf(nB, cm[2], acc.m[2]);
    acc.m[3] = fmaf(nB, cm[3], acc.m[3]);
}

// Eight Q4_0 blocks (src/quant.cpp:331-339), one activation row. A block is a 2-byte scale d and 16 bytes whose
// low nibbles are quants 0..15 and whose high nibbles are quants 16..31; the value is d * (q - 8). Per block two
// k16 MMAs over the same 16 bytes, L = (bytes & 0x0F) and R = raw bytes, against columns [limb j over the low
// half, limb j over the high half]: low half = L[even column], high half = (R[odd] - L[odd]) / 16. Lane t keeps
// limb t of rows g and g+8 (times 16); lane t = 3, whose columns carry no limb, keeps d * (sum of X over the
// block) instead, which enters the result with weight -8. Blocks at an even index have their quants 2 bytes off
// a word boundary: lane t = 0 glues the half words at the two ends (the limbs are laid out to match).
__device__ __forceinline__ void unit_q4_0(const uint8_t *rowA, const uint8_t *rowB, const int8_t *bq, const float *fs, int t,
                                          AccumSingle &acc) {
#pragma unroll
    for (int b = 0; b < 8; b++) {
        uint32_t qa, qb;
        float dA, dB;
        if ((b & 1) == 0) {
            const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowA + 18 * b);
            const uint32_t *wb = reinterpret_cast<const uint32_t *>(rowB + 18 * b);
            const uint32_t a_first = wa[0], b_first = wb[0];
            qa = t == 0 ? __byte_perm(a_first, wa[4], 0x5432) : wa[t];
            qb = t == 0 ? __byte_perm(b_first, wb[4], 0x5432) : wb[t];
            dA = half_lo(a_first);
            dB = half_lo(b_first);
        } else {
            qa = reinterpret_cast<const uint32_t *>(rowA + 18 * b + 2)[t];
            qb = reinterpret_cast<const uint32_t *>(rowB + 18 * b + 2)[t];
            dA = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowA + 18 * b)));
            dB = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowB + 18 * b)));
        }
        const uint32_t bw = *reinterpret_cast<const uint32_t *>(bq + 32 * b + 4 * t);
        int cl[4], cr[4];
        mma_u8_k16(cl, qa & 0x0F0F0F0Fu, qb & 0x0F0F0F0Fu, bw);
        mma_u8_k16(cr, qa, qb, bw);
        // |16 lo + hr - hl| < 2^21: 16 x (16 * 15 + 255 + 15) x 128, so the bits of 1.5 * 2^23 turn it into a float
        const int vA = 16 * cl[0] + cr[1] - cl[1], vB = 16 * cl[2] + cr[3] - cl[3];
        const float sum = fs[b];
        const float fa = t == 3 ? sum : __int_as_float(vA + 0x4B400000) - kMagic;
        const float fb = t == 3 ? sum : __int_as_float(vB + 0x4B400000) - kMagic;
        acc.f[0] = fmaf(dA, fa, acc.f[0]);
        acc.f[1] = fmaf(dB, fb, acc.f[1]);
    }
}

// The same eight blocks for 2..8 activation rows: the quants are centred first ((q + 0x78) ^ 0x80 is q - 8 as a
// signed byte, no carry since q <= 15), low and high nibbles go to one k16 MMA each per column group, and the
// columns carry the limbs of two activation rows as in the other general forms.
template <int NG>
__device__ __forceinline__ void unit_q4_0_rows(const uint8_t *rowA, const uint8_t *rowB, int kbase, const int8_t *const (&bp)[NG],
                                               int t, Accum<NG> &acc) {
#pragma unroll
    for (int b = 0; b < 8; b++) {
        uint32_t qa, qb;
        float dA, dB;
        if ((b & 1) == 0) {
            const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowA + 18 * b);
            const uint32_t *wb = reinterpret_cast<const uint32_t *>(rowB + 18 * b);
            const uint32_t a_first = wa[0], b_first = wb[0];
            qa = t == 0 ? __byte_perm(a_first, wa[4], 0x5432) : wa[t];
            qb = t == 0 ? __byte_perm(b_first, wb[4], 0x5432) : wb[t];
            dA = half_lo(a_first);
            dB = half_lo(b_first);
        } else {
            qa = reinterpret_cast<const uint32_t *>(rowA + 18 * b + 2)[t];
            qb = reinterpret_cast<const uint32_t *>(rowB + 18 * b + 2)[t];
            dA = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowA + 18 * b)));
            dB = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowB + 18 * b)));
        }
        // The A operand is 16 * (q - 8) as a signed byte: the nibble in the high half of the byte with its top bit
        // flipped (one instruction for the high nibbles, a shift more for the low ones); the 16 leaves with d.
        // Both MMAs of a block add onto one accumulator preset to the bits of 1.5 * 2^23, whose bits read as a
        // float are that plus the sum (|sum| <= 32 * 128 * 128 = 2^19), so the int-to-float step is a subtraction.
        const uint32_t la = ((qa << 4) & 0xF0F0F0F0u) ^ 0x80808080u, lb = ((qb << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
        const uint32_t ha = (qa & 0xF0F0F0F0u) ^ 0x80808080u, hb = (qb & 0xF0F0F0F0u) ^ 0x80808080u;
        dA *= 0.0625f;
        dB *= 0.0625f;
#pragma unroll
        for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 4 * t);
            const uint32_t b1 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 16 + 4 * t);
            int c[4] = {0x4B400000, 0x4B400000, 0x4B400000, 0x4B400000};
            mma_s8_k16_chain(c, la, lb, b0);
            mma_s8_k16_chain(c, ha, hb, b1);
            acc.f[mg][0] = fmaf(dA, __int_as_float(c[0]) - kMagic, acc.f[mg][0]);
            acc.f[mg][1] = fmaf(dA, __int_as_float(c[1]) - kMagic, acc.f[mg][1]);
            acc.f[mg][2] = fmaf(dB, __int_as_float(c[2]) - kMagic, acc.f[mg][2]);
            acc.f[mg][3] = fmaf(dB, __int_as_float(c[3]) - kMagic, acc.f[mg][3]);
        }
    }
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Eight IQ4_NL blocks (src/quant.cpp:88-91, 566-575): Q4_0's layout, but a nibble is an index into a grid of 16
// signed bytes. The grid lies in four words; a byte permute looks four indices up in two of them at a time (the
// low three bits of each nibble of the selector), once in the lower and once in the upper half of the grid, and
// the index's top bit picks between the two through a mask made by another permute in its sign-replicating mode.
// Nibbles 0..3 of a quant word are [low 0, high 0, low 1, high 1], so two last permutes regroup the results into
// the four low-nibble and the four high-nibble values. 13 integer instructions per eight values. The limbs lie
// as for Q4_0.
template <int NG>
__device__ __forceinline__ void unit_iq4_nl(const uint8_t *rowA, const uint8_t *rowB, int kbase, const int8_t *const (&bp)[NG],
                                            int t, Accum<NG> &acc) {
    constexpr uint32_t kG0 = 0xBFAD9881u, kG1 = 0xF6EADDCFu, kG2 = 0x26190D01u, kG3 = 0x71594535u;
    auto grid = [&](uint32_t q, uint32_t &lo4, uint32_t &hi4) {
        const uint32_t s = q & 0x77777777u, s2 = s >> 16, y = q << 4;
        const uint32_t m01 = prmt(y, q, 0xD9C8u), m23 = prmt(y, q, 0xFBEAu);   // 0xFF where the index is 8..15
        const uint32_t r01 = (prmt(kG0, kG1, s) & ~m01) | (prmt(kG2, kG3, s) & m01);
        const uint32_t r23 = (prmt(kG0, kG1, s2) & ~m23) | (prmt(kG2, kG3, s2) & m23);
        lo4 = prmt(r01, r23, 0x6420u);
        hi4 = prmt(r01, r23, 0x7531u);
    };
#pragma unroll
    for (int b = 0; b < 8; b++) {
        uint32_t qa, qb;
        float dA, dB;
        if ((b & 1) == 0) {
            const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowA + 18 * b);
            const uint32_t *wb = reinterpret_cast<const uint32_t *>(rowB + 18 * b);
            const uint32_t a_first = wa[0], b_first = wb[0];
            qa = t == 0 ? __byte_perm(a_first, wa[4], 0x5432) : wa[t];
            qb = t == 0 ? __byte_perm(b_first, wb[4], 0x5432) : wb[t];
            dA = half_lo(a_first);
            dB = half_lo(b_first);
        } else {
            qa = reinterpret_cast<const uint32_t *>(rowA + 18 * b + 2)[t];
            qb = reinterpret_cast<const uint32_t *>(rowB + 18 * b + 2)[t];
            dA = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowA + 18 * b)));
            dB = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowB + 18 * b)));
        }
        uint32_t la, ha, lb, hb;
        grid(qa, la, ha);
        grid(qb, lb, hb);
#pragma unroll
        for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 4 * t);
            const uint32_t b1 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 16 + 4 * t);
            int c[4] = {0x4B400000, 0x4B400000, 0x4B400000, 0x4B400000};   // |sum| <= 32 * 127 * 128 < 2^19
            mma_s8_k16_chain(c, la, lb, b0);
            mma_s8_k16_chain(c, ha, hb, b1);
            acc.f[mg][0] = fmaf(dA, __int_as_float(c[0]) - kMagic, acc.f[mg][0]);
            acc.f[mg][1] = fmaf(dA, __int_as_float(c[1]) - kMagic, acc.f[mg][1]);
            acc.f[mg][2] = fmaf(dB, __int_as_float(c[2]) - kMagic, acc.f[mg][2]);
            acc.f[mg][3] = fmaf(dB, __int_as_float(c[3]) - kMagic, acc.f[mg][3]);
        }
    }
}

// Bits 0..3 of n to bit 7 of bytes 0..3: bit i times 2^(7j + 7) lands at 8k + 7 only for i = j = k, and no two
// products share a position, so nothing carries.
__device__ __forceinline__ uint32_t spread_top(uint32_t n) { return (n * 0x10204080u) & 0x80808080u; }

// Eight Q5_0 blocks (src/quant.cpp:352-364): a 2-byte scale d, a 32-bit mask of fifth bits, 16 bytes whose low
// nibbles are quants 0..15 and whose high nibbles are quants 16..31; the value is d * (q - 16). The A operand is
// 8 * (q - 16) as a signed byte: the nibble at bits 3-6 and the inverted fifth bit at bit 7 (q - 16 is q with
// bit 4 flipped, read as a 5-bit two's complement); the 8 leaves with d. Two k16 MMAs per block and column
// group, chained on one accumulator preset to the bits of 1.5 * 2^23 (|sum| <= 32 * 128 * 128 = 2^19). Blocks at
// an even index have mask and quants 2 bytes off a word boundary: the mask is glued from two words, lane t takes
// quant bytes 4t-2..4t+1 (lane 0: 14, 15, 0, 1) and the mask is rotated to match.
template <int NG>
__device__ __forceinline__ void unit_q5_0(const uint8_t *rowA, const uint8_t *rowB, int kbase, const int8_t *const (&bp)[NG],
                                          int t, Accum<NG> &acc) {
#pragma unroll
    for (int b = 0; b < 8; b++) {
        uint32_t qa, qb, ma, mb;
        float dA, dB;
        if ((b & 1) == 0) {
            const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowA + 22 * b);
            const uint32_t *wb = reinterpret_cast<const uint32_t *>(rowB + 22 * b);
            const uint32_t a0 = wa[0], a1 = wa[1], b0 = wb[0], b1 = wb[1];
            qa = t == 0 ? __byte_perm(a1, wa[5], 0x3254) : wa[t + 1];
            qb = t == 0 ? __byte_perm(b1, wb[5], 0x3254) : wb[t + 1];
            const uint32_t ha = ~__byte_perm(a0, a1, 0x5432), hb = ~__byte_perm(b0, b1, 0x5432);
            ma = ((ha << 2) & 0xFFFCFFFCu) | ((ha >> 14) & 0x00030003u);   // both 16-bit halves rotated left by 2
            mb = ((hb << 2) & 0xFFFCFFFCu) | ((hb >> 14) & 0x00030003u);
            dA = half_lo(a0);
            dB = half_lo(b0);
        } else {
            qa = reinterpret_cast<const uint32_t *>(rowA + 22 * b + 6)[t];
            qb = reinterpret_cast<const uint32_t *>(rowB + 22 * b + 6)[t];
            ma = ~*reinterpret_cast<const uint32_t *>(rowA + 22 * b + 2);
            mb = ~*reinterpret_cast<const uint32_t *>(rowB + 22 * b + 2);
            dA = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowA + 22 * b)));
            dB = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowB + 22 * b)));
        }
        const uint32_t la = ((qa << 3) & 0x78787878u) | spread_top((ma >> (4 * t)) & 0xFu);
        const uint32_t lb = ((qb << 3) & 0x78787878u) | spread_top((mb >> (4 * t)) & 0xFu);
        const uint32_t ha = ((qa >> 1) & 0x78787878u) | spread_top((ma >> (16 + 4 * t)) & 0xFu);
        const uint32_t hb = ((qb >> 1) & 0x78787878u) | spread_top((mb >> (16 + 4 * t)) & 0xFu);
        dA *= 0.125f;
        dB *= 0.125f;
#pragma unroll
        for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 4 * t);
            const uint32_t b1 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 16 + 4 * t);
            int c[4] = {0x4B400000, 0x4B400000, 0x4B400000, 0x4B400000};
            mma_s8_k16_chain(c, la, lb, b0);
            mma_s8_k16_chain(c, ha, hb, b1);
            acc.f[mg][0] = fmaf(dA, __int_as_float(c[0]) - kMagic, acc.f[mg][0]);
            acc.f[mg][1] = fmaf(dA, __int_as_float(c[1]) - kMagic, acc.f[mg][1]);
            acc.f[mg][2] = fmaf(dB, __int_as_float(c[2]) - kMagic, acc.f[mg][2]);
            acc.f[mg][3] = fmaf(dB, __int_as_float(c[3]) - kMagic, acc.f[mg][3]);
        }
    }
}

// Eight Q5_1 blocks (src/quant.cpp:366-379): scale d, offset m, the mask, the nibbles, all on word boundaries;
// the value is d * q + m with q = 0..31. The A operand is 8 * q as an unsigned byte; the offset enters as
// m * (sum of X over the block), which the activation pass leaves per block as a float: the lanes whose columns
// carry the limb of weight 1 (column 2 of the even, column 5 of the odd activation row of a group) add it.
template <int NG>
__device__ __forceinline__ void unit_q5_1(const uint8_t *rowA, const uint8_t *rowB, int kbase, const int8_t *const (&bp)[NG],
                                          const float *const (&fe)[NG], const float *const (&fo)[NG], int t, Accum<NG> &acc) {
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowA + 24 * b);
        const uint32_t *wb = reinterpret_cast<const uint32_t *>(rowB + 24 * b);
        const uint32_t a0 = wa[0], b0w = wb[0], ma = wa[1], mb = wb[1], qa = wa[2 + t], qb = wb[2 + t];
        const float dA = 0.125f * half_lo(a0), dB = 0.125f * half_lo(b0w), oA = half_hi(a0), oB = half_hi(b0w);
        const uint32_t la = ((qa << 3) & 0x78787878u) | spread_top((ma >> (4 * t)) & 0xFu);
        const uint32_t lb = ((qb << 3) & 0x78787878u) | spread_top((mb >> (4 * t)) & 0xFu);
        const uint32_t ha = ((qa >> 1) & 0x78787878u) | spread_top((ma >> (16 + 4 * t)) & 0xFu);
        const uint32_t hb = ((qb >> 1) & 0x78787878u) | spread_top((mb >> (16 + 4 * t)) & 0xFu);
#pragma unroll
        for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 4 * t);
            const uint32_t b1 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 16 + 4 * t);
            int c[4] = {0x4B400000, 0x4B400000, 0x4B400000, 0x4B400000};   // |sum| <= 32 * 248 * 128 < 2^20
            mma_u8_k16_chain(c, la, lb, b0);
            mma_u8_k16_chain(c, ha, hb, b1);
            // (five to eight rows: the weight-1 limbs of rows 6 and 7 are columns 6 and 7 of group 2, in lane t = 3)
            const bool spare = NG == 4 && mg == 2 && t == 3;
            const float se = t == 1 ? fe[mg][(kbase >> 5) + b] : (spare ? fe[NG - 1][(kbase >> 5) + b] : 0.0f);
            const float so = t == 2 ? fo[mg][(kbase >> 5) + b] : (spare ? fo[NG - 1][(kbase >> 5) + b] : 0.0f);
            acc.f[mg][0] = fmaf(dA, __int_as_float(c[0]) - kMagic, fmaf(oA, se, acc.f[mg][0]));
            acc.f[mg][1] = fmaf(dA, __int_as_float(c[1]) - kMagic, fmaf(oA, so, acc.f[mg][1]));
            acc.f[mg][2] = fmaf(dB, __int_as_float(c[2]) - kMagic, fmaf(oB, se, acc.f[mg][2]));
            acc.f[mg][3] = fmaf(dB, __int_as_float(c[3]) - kMagic, fmaf(oB, so, acc.f[mg][3]));
        }
    }
}

// Four Q8_0 blocks. A block is a 2-byte scale then 32 quants, so blocks at an even index have
// their quants 2 bytes off a word boundary: their lanes read the aligned words and lane t = 0
// glues the two half words at the ends into one (the activation limbs are permuted to match).
template <int NG>
__device__ __forceinline__ void unit_q8_0(const uint8_t *rowA, const uint8_t *rowB, int kbase, const int8_t *const (&bp)[NG],
                                          int t, Accum<NG> &acc) {
#pragma unroll
    for (int b = 0; b < 4; b++) {
        uint32_t a0, a1, a2, a3;
        float dA, dB;
        if ((b & 1) == 0) {
            const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowA + 34 * b);
            const uint32_t *wb = reinterpret_cast<const uint32_t *>(rowB + 34 * b);
            const uint32_t a_first = wa[0], b_first = wb[0];
            a0 = t == 0 ? __byte_perm(a_first, wa[8], 0x5432) : wa[t];
            a1 = t == 0 ? __byte_perm(b_first, wb[8], 0x5432) : wb[t];
            a2 = wa[t + 4];
            a3 = wb[t + 4];
            dA = half_lo(a_first);
            dB = half_lo(b_first);
        } else {
            const uint32_t *wa = reinterpret_cast<const uint32_t *>(rowA + 34 * b + 2);
            const uint32_t *wb = reinterpret_cast<const uint32_t *>(rowB + 34 * b + 2);
            a0 = wa[t];
            a1 = wb[t];
            a2 = wa[t + 4];
            a3 = wb[t + 4];
            dA = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowA + 34 * b)));
            dB = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rowB + 34 * b)));
        }
#pragma unroll
        for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 4 * t);
            const uint32_t b1 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 32 * b + 16 + 4 * t);
            int cc[4];   // (presetting the accumulator to 1.5 * 2^23 to save the int-to-float step is 0.3-3 % slower here)
            mma_s8_k32(cc, a0, a1, a2, a3, b0, b1);
            acc.f[mg][0] = fmaf(dA, (float)cc[0], acc.f[mg][0]);
            acc.f[mg][1] = fmaf(dA, (float)cc[1], acc.f[mg][1]);
            acc.f[mg][2] = fmaf(dB, (float)cc[2], acc.f[mg][2]);
            acc.f[mg][3] = fmaf(dB, (float)cc[3], acc.f[mg][3]);
        }
    }
}

// 32-bit load at a 4-byte-multiple offset of a Q6_K block that itself starts 0 or 2 bytes off
// a word boundary (blocks are 210 bytes, so odd blocks of a row are misaligned).
// MODE 0: the block starts on a word boundary; 1: 2 bytes off; 2: either, found from the address (ragged rows:
// the two rows of a lane may differ).
template <int MODE>
__device__ __forceinline__ uint32_t ld_q6(const uint8_t *blk, int off) {
    if (MODE == 2) {
        const uintptr_t a = reinterpret_cast<uintptr_t>(blk + off);
        const uint32_t *w = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
        return __funnelshift_r(w[0], w[1], (uint32_t)(a & 2) * 8u);
    }
    if (MODE == 1) {
        const uint32_t lo = *reinterpret_cast<const uint32_t *>(blk + off - 2);
        const uint32_t hi = *reinterpret_cast<const uint32_t *>(blk + off + 2);
        return __byte_perm(lo, hi, 0x5432);
    }
    return *reinterpret_cast<const uint32_t *>(blk + off);
}

// The A operand is 4 * (q - 32) as a signed byte: the low four quant bits at bits 2-5, the high two at bits 6-7
// with the top one flipped (q - 32 is q with bit 5 flipped, read as a 6-bit two's complement; at the top of the
// byte it needs no sign extension). The flip is done once per word of high bits, before the fields are split.
// Four integer instructions per four quants against six for assembling q and then centring it; the factor 4
// leaves with the block scale.

template <int NG, int ODD>
__device__ __forceinline__ void unit_q6_k(const uint8_t *blkA, const uint8_t *blkB, int kbase, const int8_t *const (&bp)[NG],
                                          int t, Accum<NG> &acc) {
    int I[NG][4];
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++)
#pragma unroll
        for (int j = 0; j < 4; j++) I[mg][j] = 0;
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint32_t qlA[4], qlB[4], qhA[2], qhB[2], scA[2], scB[2];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            qlA[i] = ld_q6<ODD>(blkA, 64 * h + 16 * i + 4 * t);
            qlB[i] = ld_q6<ODD>(blkB, 64 * h + 16 * i + 4 * t);
        }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            qhA[i] = ld_q6<ODD>(blkA, 128 + 32 * h + 16 * i + 4 * t) ^ 0xAAAAAAAAu;
            qhB[i] = ld_q6<ODD>(blkB, 128 + 32 * h + 16 * i + 4 * t) ^ 0xAAAAAAAAu;
            scA[i] = ld_q6<ODD>(blkA, 192 + 8 * h + 4 * i);
            scB[i] = ld_q6<ODD>(blkB, 192 + 8 * h + 4 * i);
        }
        // group G = 2*quad + s covers values 16G..16G+15 of the half (src/quant.cpp:491-512):
        // low 4 bits from ql[32*(quad&1) + 16s ...] (high nibble when quad >= 2), bits 4-5 from
        // qh[16s ...] >> 2*quad.
#pragma unroll
        for (int G = 0; G < 8; G++) {
            const int quad = G >> 1, s = G & 1;
            const uint32_t la = qlA[2 * (quad & 1) + s], lb = qlB[2 * (quad & 1) + s];
            const uint32_t lowA = (quad & 2) ? (la >> 2) : shl_mad<4u>(la);
            const uint32_t lowB = (quad & 2) ? (lb >> 2) : shl_mad<4u>(lb);
            const uint32_t hiA = quad == 0 ? shl_mad<64u>(qhA[s]) : quad == 1 ? shl_mad<16u>(qhA[s]) : quad == 2 ? shl_mad<4u>(qhA[s]) : qhA[s];
            const uint32_t hiB = quad == 0 ? shl_mad<64u>(qhB[s]) : quad == 1 ? shl_mad<16u>(qhB[s]) : quad == 2 ? shl_mad<4u>(qhB[s]) : qhB[s];
            const uint32_t a0 = (lowA & 0x3C3C3C3Cu) | (hiA & 0xC0C0C0C0u);
            const uint32_t a1 = (lowB & 0x3C3C3C3Cu) | (hiB & 0xC0C0C0C0u);
            const int sa = sext_byte(scA[G >> 2], G & 3), sb = sext_byte(scB[G >> 2], G & 3);
#pragma unroll
            for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 128 * h + 16 * G + 4 * t);
                int cc[4];
                mma_s8_k16(cc, a0, a1, b0);
                I[mg][0] += sa * cc[0];
                I[mg][1] += sa * cc[1];
                I[mg][2] += sb * cc[2];
                I[mg][3] += sb * cc[3];
            }
        }
    }
    const float dA = 0.25f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blkA + 208)));
    const float dB = 0.25f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blkB + 208)));
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
        acc.f[mg][0] = fmaf(dA, (float)I[mg][0], acc.f[mg][0]);
        acc.f[mg][1] = fmaf(dA, (float)I[mg][1], acc.f[mg][1]);
        acc.f[mg][2] = fmaf(dB, (float)I[mg][2], acc.f[mg][2]);
        acc.f[mg][3] = fmaf(dB, (float)I[mg][3], acc.f[mg][3]);
    }
}

// A Q2_K super-block (src/quant.cpp:398-424): 16 bytes of (scale | min << 4), 64 bytes of 2-bit quants, d, dmin;
// value = d * scale * q - dmin * min per group of 16. Blocks are 84 bytes, so every word load is aligned. Group
// G = 8n + 2j + s takes bits 2j, 2j+1 of quant bytes 32n + 16s ..+15: one shift and one AND per four quants, one
// k16 MMA per group. The minimums go through one more MMA per super-block, the 16 of them against the group
// sums of X (acc.m, as for Q4_K).
template <int NG>
__device__ __forceinline__ void unit_q2_k(const uint8_t *blkA, const uint8_t *blkB, int kbase, const int8_t *const (&bp)[NG],
                                          const int8_t *const (&sp)[NG], int t, Accum<NG> &acc) {
    const uint32_t *wa = reinterpret_cast<const uint32_t *>(blkA), *wb = reinterpret_cast<const uint32_t *>(blkB);
    uint32_t scA[4], scB[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        scA[k] = wa[k];
        scB[k] = wb[k];
    }
    int I[NG][4];
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++)
#pragma unroll
        for (int j = 0; j < 4; j++) I[mg][j] = 0;
#pragma unroll
    for (int n = 0; n < 2; n++) {
        const uint32_t qA[2] = {wa[4 + 8 * n + t], wa[8 + 8 * n + t]}, qB[2] = {wb[4 + 8 * n + t], wb[8 + 8 * n + t]};
#pragma unroll
        for (int js = 0; js < 8; js++) {
            const int j = js >> 1, s = js & 1, G = 8 * n + js;
            const uint32_t a0 = (qA[s] >> (2 * j)) & 0x03030303u, a1 = (qB[s] >> (2 * j)) & 0x03030303u;
            const int sa = (scA[G >> 2] >> (8 * (G & 3))) & 0xF, sb = (scB[G >> 2] >> (8 * (G & 3))) & 0xF;
#pragma unroll
            for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 16 * G + 4 * t);
                int cc[4];
                mma_s8_k16(cc, a0, a1, b0);
                I[mg][0] += sa * cc[0];
                I[mg][1] += sa * cc[1];
                I[mg][2] += sb * cc[2];
                I[mg][3] += sb * cc[3];
            }
        }
    }
    const uint32_t hA = wa[20], hB = wb[20];
    const float dA = half_lo(hA), dB = half_lo(hB), nA = half_hi(hA), nB = half_hi(hB);
    const uint32_t m0 = (wa[t] >> 4) & 0x0F0F0F0Fu, m1 = (wb[t] >> 4) & 0x0F0F0F0Fu;   // k slot j = group j: lane t brings 4t..4t+3
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
        acc.f[mg][0] = fmaf(dA, (float)I[mg][0], acc.f[mg][0]);
        acc.f[mg][1] = fmaf(dA, (float)I[mg][1], acc.f[mg][1]);
        acc.f[mg][2] = fmaf(dB, (float)I[mg][2], acc.f[mg][2]);
        acc.f[mg][3] = fmaf(dB, (float)I[mg][3], acc.f[mg][3]);
    }
#pragma unroll
    for (int mg = 0; mg < NG; mg++) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(sp[mg] + (kbase >> 4) + 4 * t);
        int cc[4];
        mma_s8_k16(cc, m0, m1, b0);
        acc.m[mg][0] = fmaf(nA, (float)cc[0], acc.m[mg][0]);
        acc.m[mg][1] = fmaf(nA, (float)cc[1], acc.m[mg][1]);
        acc.m[mg][2] = fmaf(nB, (float)cc[2], acc.m[mg][2]);
        acc.m[mg][3] = fmaf(nB, (float)cc[3], acc.m[mg][3]);
    }
}

// A Q3_K super-block (src/quant.cpp:514-553): 32 mask bytes, 64 bytes of 2-bit quants, sixteen 6-bit scales in 12
// bytes, d; value = d * (scale - 32) * (q2 - (mask bit ? 0 : 4)). The A operand is 32 * (q3 - 4) with q3 = q2 + 4 *
// mask bit: q2 at bits 5-6 and the inverted mask bit at bit 7 (a 3-bit two's complement at the top of the byte),
// two shifts, an AND and an AND-OR per four quants; the 32 leaves with d. Blocks are 110 bytes: every other one is
// 2 bytes off a word boundary (MODE as for Q6_K).
template <int NG, int MODE>
__device__ __forceinline__ void unit_q3_k(const uint8_t *blkA, const uint8_t *blkB, int kbase, const int8_t *const (&bp)[NG],
                                          int t, Accum<NG> &acc) {
    uint32_t SA[4], SB[4];
    {
        const uint32_t a0 = ld_q6<MODE>(blkA, 96), a1 = ld_q6<MODE>(blkA, 100), a2 = ld_q6<MODE>(blkA, 104);
        const uint32_t b0 = ld_q6<MODE>(blkB, 96), b1 = ld_q6<MODE>(blkB, 100), b2 = ld_q6<MODE>(blkB, 104);
        // scale i: low four bits in the nibbles of bytes 0..7, high two in byte 8 + i % 4 at bits 2 * (i / 4)
        SA[0] = (a0 & 0x0F0F0F0Fu) | ((a2 << 4) & 0x30303030u);
        SA[1] = (a1 & 0x0F0F0F0Fu) | ((a2 << 2) & 0x30303030u);
        SA[2] = ((a0 >> 4) & 0x0F0F0F0Fu) | (a2 & 0x30303030u);
        SA[3] = ((a1 >> 4) & 0x0F0F0F0Fu) | ((a2 >> 2) & 0x30303030u);
        SB[0] = (b0 & 0x0F0F0F0Fu) | ((b2 << 4) & 0x30303030u);
        SB[1] = (b1 & 0x0F0F0F0Fu) | ((b2 << 2) & 0x30303030u);
        SB[2] = ((b0 >> 4) & 0x0F0F0F0Fu) | (b2 & 0x30303030u);
        SB[3] = ((b1 >> 4) & 0x0F0F0F0Fu) | ((b2 >> 2) & 0x30303030u);
#pragma unroll
        for (int k = 0; k < 4; k++) {   // scale - 32 as signed bytes: add 0x60 (no carry: scale <= 63), flip the sign bit
            SA[k] = (SA[k] + 0x60606060u) ^ 0x80808080u;
            SB[k] = (SB[k] + 0x60606060u) ^ 0x80808080u;
        }
    }
    const uint32_t hmA[2] = {~ld_q6<MODE>(blkA, 4 * t), ~ld_q6<MODE>(blkA, 16 + 4 * t)};
    const uint32_t hmB[2] = {~ld_q6<MODE>(blkB, 4 * t), ~ld_q6<MODE>(blkB, 16 + 4 * t)};
    int I[NG][4];
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++)
#pragma unroll
        for (int j = 0; j < 4; j++) I[mg][j] = 0;
#pragma unroll
    for (int n = 0; n < 2; n++) {
        const uint32_t qA[2] = {ld_q6<MODE>(blkA, 32 + 32 * n + 4 * t), ld_q6<MODE>(blkA, 48 + 32 * n + 4 * t)};
        const uint32_t qB[2] = {ld_q6<MODE>(blkB, 32 + 32 * n + 4 * t), ld_q6<MODE>(blkB, 48 + 32 * n + 4 * t)};
#pragma unroll
        for (int js = 0; js < 8; js++) {
            const int j = js >> 1, s = js & 1, G = 8 * n + js, hb = 4 * n + j;
            const uint32_t qa = j < 3 ? (qA[s] << (5 - 2 * j)) : (qA[s] >> 1), qb = j < 3 ? (qB[s] << (5 - 2 * j)) : (qB[s] >> 1);
            const uint32_t a0 = (qa & 0x60606060u) | ((hmA[s] << (7 - hb)) & 0x80808080u);
            const uint32_t a1 = (qb & 0x60606060u) | ((hmB[s] << (7 - hb)) & 0x80808080u);
            const int sa = sext_byte(SA[G >> 2], G & 3), sb = sext_byte(SB[G >> 2], G & 3);
#pragma unroll
            for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(bp[mg] + kbase + 16 * G + 4 * t);
                int cc[4];
                mma_s8_k16(cc, a0, a1, b0);
                I[mg][0] += sa * cc[0];
                I[mg][1] += sa * cc[1];
                I[mg][2] += sb * cc[2];
                I[mg][3] += sb * cc[3];
            }
        }
    }
    const float dA = 0.03125f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blkA + 108)));
    const float dB = 0.03125f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blkB + 108)));
#pragma unroll
    for (int mg = 0; mg < kMmaGroups<NG>; mg++) {
        acc.f[mg][0] = fmaf(dA, (float)I[mg][0], acc.f[mg][0]);
        acc.f[mg][1] = fmaf(dA, (float)I[mg][1], acc.f[mg][1]);
        acc.f[mg][2] = fmaf(dB, (float)I[mg][2], acc.f[mg][2]);
        acc.f[mg][3] = fmaf(dB, (float)I[mg][3], acc.f[mg][3]);
    }
}

// ---- the kernel ------------------------------------------------------------------------------------------
// Three roles, connected only by mbarriers, so no warp ever waits at a CTA-wide barrier while
// weights are streaming:
//   warp 0        producer: bulk-async copies of weight rows into the stage ring. It is the first warp of
//                 the CTA to run, sets the barriers up itself and issues its first copies without waiting
//                 for the other warps to start;
//   warps 1..8    consumers: warp w takes K unit w of every stage (16 rows x 256 values), keeps the
//                 tile's partial sums in registers and hands them over at the end of the tile;
//   warp 9        epilogue: adds the partial sums of each tile in warp order (deterministic),
//                 applies the gate/up fold or the residual add, and writes y.

// SINGLE: 0 the general form; 1 Q4_K with one activation row (unit_q4_k_single); 2 the same with the B
// fragments of the warp's (at most two) K units held in registers, for rows of at most 16 units.
// Two CTAs per SM (96 registers per thread) or one (up to 192). One or two activation rows always fit in 96.
// Three or four rows (two column groups) of Q8_0 also do, and two half-SM CTAs are then 1.1-1.5x faster than one
// at every size. Q4_0 fits too but gains only on very tall matrices (+14 % at 131072 rows, -3 to -9 % at layer
// sizes); the K-quant forms spill at 96 registers and are faster alone on an SM at layer sizes.
template <int WT, int NG>
constexpr bool kTwoPerSm = NG == 1 || (NG == 2 && WT == KRK_CUDA_Q8_0);

// RAG: the form for ragged rows of Q6_K and Q3_K, whose units find each word's alignment from its address; compiled
// apart so that the usual form does not carry a third copy of the unit.
template <int WT, int NG, bool STACK, int SINGLE, bool RAG = false>
__global__ void __launch_bounds__(kThreads, kTwoPerSm<WT, NG> ? 2 : 1)
gemv_stream_kernel(const __grid_constant__ StreamParams p) {
    // STACK: several 16-row tiles per stage (p.tps of them); compiled apart so that the usual one-tile
    // form carries none of its index arithmetic.
    static_assert(!SINGLE || ((WT == KRK_CUDA_Q4_K || WT == KRK_CUDA_Q4_0) && NG == 1), "the single-row forms are Q4_K and Q4_0");
    const int tps = STACK ? p.tps : 1;
    using F = Fmt<WT>;
    using SmemT = Smem<NG>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    SmemT *sm = reinterpret_cast<SmemT *>(smem_raw);
    int8_t *planes = reinterpret_cast<int8_t *>(smem_raw + align_up((int)sizeof(SmemT), 128));
    // one copy of the prepared activation per stacked sub-tile: the warps of a sub-tile move on to the next
    // matrix (and its activation) on their own, so they must not share planes with another sub-tile
    int8_t *chunk_sum = planes + tps * plane_bytes<WT>(p.n_in, p.rows);
    uint8_t *stages = reinterpret_cast<uint8_t *>(chunk_sum) + tps * chunk_sum_bytes<WT>(p.n_in, p.rows);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_warps = min(kConsumerWarps, p.units * tps);   // consumer warps that ever hold a unit
    const int sub_warps = STACK ? p.units : n_warps;         // warps that share one 16-row tile
    // Programmatic dependent launch: the next kernel in the stream may become resident beside this one
    // (a CTA takes half an SM) as soon as every CTA here has passed this point; it prefetches weights
    // and waits for this grid to complete before touching activations or outputs.
    if (!(p.tune & 2)) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    volatile int *gave_up = &sm->gave_up;

    if (warp == 0) {
        // ===== producer warp: weights only, so it can run ahead of everything else =====
        if (lane == 0) {
            for (int s = 0; s < p.n_stages; s++) {
                mbar_init(smem_u32(&sm->full[s]), 1);
                mbar_init(smem_u32(&sm->empty[s]), kConsumerWarps);
            }
            for (int s = 0; s < red_slots(NG); s++) {
                mbar_init(smem_u32(&sm->red_full[s]), n_warps);
                mbar_init(smem_u32(&sm->red_empty[s]), 1);
            }
            sm->gave_up = 0;
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __threadfence_block();
        }
        __syncwarp();
        // the other warps wait here for the barriers (they arrive as they start); this warp does not wait
        asm volatile("bar.arrive 1, %0;" ::"r"(kThreads) : "memory");
        // A device-side table is the output of the kernel before this one: wait for that grid.
        if (p.dev_table || (p.tune & 1)) asm volatile("griddepcontrol.wait;" ::: "memory");
        const TableView tv = table_view(p);
        walk(p, tv, tps, [](int) {}, [&](const StageInfo &s) {
            const int slot = s.slot;
            const uint32_t full = smem_u32(&sm->full[slot]), empty = smem_u32(&sm->empty[slot]);
            wait_phase(empty, s.phase ^ 1, gave_up, p.status);
            uint8_t *dst = stages + (size_t)slot * p.stage_bytes;
            const uint8_t *src = tv.mat[s.mat].w + (size_t)s.row0 * p.row_bytes;
            if (p.use_tma) {
                // the box is clipped where the matrix ends (rows past n_out, units past the row) and
                // still signals its full size
                if (lane == 0) {
                    mbar_arrive_expect_tx(full, (uint32_t)p.box_bytes);
                    if (p.dev_table) {
                        // (a 64-bit division per stage, by the one lane that issues a copy per stage)
                        const int bank = s.mat % p.step;
                        const int row_off = (int)((size_t)(tv.mat[s.mat].w - p.bank_base[bank]) / (size_t)p.row_bytes);
                        tma_box(smem_u32(dst), &p.wmap[bank], row_off + s.row0, s.unit0 / p.tma_unit_div, full);
                    } else {
                        tma_box(smem_u32(dst), &p.wmap[s.mat], s.row0, s.unit0 / p.tma_unit_div, full);
                    }
                }
            } else if ((WT == KRK_CUDA_Q6_K || WT == KRK_CUDA_Q2_K || WT == KRK_CUDA_Q3_K) && p.ragged) {
                // a stage starts a multiple of 8 units (a multiple of 16 bytes in all three formats) into its rows, so a row lies equally far off
                // a 16-byte boundary in every stage
                const uint32_t bytes = (uint32_t)s.n_units * F::unit_bytes;
                uint32_t total = 0;
                for (int r = lane; r < s.n_rows; r += 32) {
                    const uint32_t a = (uint32_t)(reinterpret_cast<uintptr_t>(src + (size_t)r * p.row_bytes) & 15);
                    total += (a + bytes + 15u) & ~15u;
                }
                total = __reduce_add_sync(0xFFFFFFFFu, total);
                if (lane == 0) mbar_arrive_expect_tx(full, total);
                __syncwarp();
                for (int r = lane; r < s.n_rows; r += 32) {
                    const uint8_t *row = src + (size_t)r * p.row_bytes + (size_t)s.unit0 * F::unit_bytes;
                    const uint32_t a = (uint32_t)(reinterpret_cast<uintptr_t>(row) & 15);
                    bulk_g2s(smem_u32(dst + r * p.row_stride), row - a, (a + bytes + 15u) & ~15u, full);
                }
            } else if (!p.whole_tiles) {
                const uint32_t bytes = (uint32_t)s.n_units * F::unit_bytes;
                if (lane == 0) mbar_arrive_expect_tx(full, bytes * s.n_rows);
                __syncwarp();
                for (int r = lane; r < s.n_rows; r += 32)
                    bulk_g2s(smem_u32(dst + r * p.row_stride),
                             src + (size_t)r * p.row_bytes + (size_t)s.unit0 * F::unit_bytes, bytes, full);
            } else if (lane == 0) {
                // rows are not 16-byte multiples: one copy of the whole tile, rounded down to 16 bytes,
                // and the (< 16 byte, 4-byte granular) tail with plain loads before the arrive
                const uint32_t total = (uint32_t)s.n_rows * p.row_bytes;
                const uint32_t bulk = total & ~15u;
                for (uint32_t o = bulk; o < total; o += 4)
                    *reinterpret_cast<uint32_t *>(dst + o) = *reinterpret_cast<const uint32_t *>(src + o);
                mbar_arrive_expect_tx(full, bulk);
                if (bulk) bulk_g2s(smem_u32(dst), src, bulk, full);
            }
            __syncwarp();
        });
        return;
    }
    asm volatile("bar.sync 1, %0;" ::"r"(kThreads) : "memory");
    if (p.dev_table) asm volatile("griddepcontrol.wait;" ::: "memory");
    const TableView tv = table_view(p);

    if (warp == kEpilogueWarp) {
        // ===== epilogue warp =====
        // Output (row, activation row) of a tile is the sum, over the consumer warps in warp order, of the
        // share each warp left in `red` (already added up over the four lanes of a row group).
        constexpr int kSlots = red_slots(NG);
        float gate_reg[NG];   // gate tile kept for the silu fold (stacked tiles keep theirs in shared memory)
        int tile_it = 0;
        walk(p, tv, tps, [](int) {}, [&](const StageInfo &s) {
            if (!s.last) return;
            const int slot = tile_it % kSlots;
            wait_phase(smem_u32(&sm->red_full[slot]), (tile_it / kSlots) & 1, gave_up, p.status);
            tile_it++;
#pragma unroll
            for (int sub = 0; sub < (STACK ? kMaxStack : 1); sub++) {
                if (sub >= tps) break;
#pragma unroll
                for (int i = 0; i < NG; i++) {
                    const int idx = lane + 32 * i, row = idx & (kTileRows - 1), r = idx >> 4;   // r = 2*i + (lane >> 4)
                    const float *src = reinterpret_cast<const float *>(&sm->red[slot][sub * sub_warps][i][row & 7]) +
                                       2 * (row >> 3) + (r & 1);
                    float part[kConsumerWarps];
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; w++) part[w] = w < sub_warps ? src[(size_t)w * (NG * 8 * 4)] : 0.0f;
                    float v = 0.0f;
#pragma unroll
                    for (int w = 0; w < kConsumerWarps; w++) v += part[w];
                    const int srow = kTileRows * sub + row;   // row inside the stage
                    if (r < p.rows) {
                        if (p.step == 2 && s.which == 0) {
                            if (STACK) sm->gate[sub][i][lane] = v;   // kept for the silu fold with the `up` tile
                            else gate_reg[i] = v;
                        } else if (srow < s.n_rows) {
                            if (p.n_peers > 0) {
                                // plain stores into every GPU's copy of the full row (NVLink peer stores)
                                const long long at = (long long)r * p.peer_row_stride + p.peer_offset + s.row0 + srow;
                                for (int q = 0; q < p.n_peers; q++) p.peer_y[q][at] = v;
                            } else {
                                const GemvMat &mat = tv.mat[p.step == 2 ? s.mat - 1 : s.mat];
                                float *y = mat.y + (size_t)r * mat.n_out + s.row0 + srow;
                                const float gt = STACK ? sm->gate[sub][i][lane] : gate_reg[i];
                                if (p.step == 2) v = __fmul_rn(__fdiv_rn(gt, __fadd_rn(1.0f, exp_as_host(-gt))), v);
                                *y = p.accumulate ? __fadd_rn(*y, v) : v;
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sm->red_empty[slot]));
        });
        if (p.n_peers > 0) {
            // This CTA's stores are out. The CTA that reports last publishes the epoch to every peer and
            // then waits (bounded) until every peer has published the same epoch here, so that the end
            // of this kernel is the end of the all-gather on this GPU. The count of CTAs that have
            // reported lives behind this GPU's own flags (word n_peers + 1), one per exchange object.
            __threadfence_system();
            __syncwarp();
            int *own = p.peer_flag[p.my_rank];
            unsigned *done_counter = reinterpret_cast<unsigned *>(own + p.n_peers + 1);
            unsigned done = 0;
            if (lane == 0) done = atomicAdd(done_counter, 1u);
            done = __shfl_sync(0xffffffffu, done, 0);
            if (done == gridDim.x - 1) {
                int epoch = p.epoch;
                if (lane == 0) {
                    *done_counter = 0;
                    if (epoch == 0) {   // device-counted steps: the count lives behind this GPU's flags
                        epoch = own[p.n_peers] + 1;
                        own[p.n_peers] = epoch;
                    }
                    __threadfence_system();
                    for (int q = 0; q < p.n_peers; q++) *reinterpret_cast<volatile int *>(p.peer_flag[q] + p.my_rank) = epoch;
                    __threadfence_system();
                }
                epoch = __shfl_sync(0xffffffffu, epoch, 0);
                if (p.wait_peers && lane < p.n_peers) {
                    const long long t0 = clock64();
                    while (*reinterpret_cast<const volatile int *>(own + lane) < epoch) {
                        __nanosleep(100);
                        if (clock64() - t0 > kWaitCycles) {
                            atomicExch(p.status, KRK_CUDA_ETIMEOUT);
                            break;
                        }
                    }
                }
                __threadfence_system();
            }
        }
        return;
    }

    // ===== consumer warps =====
    const int wid = warp - 1, g = lane >> 2, t = lane & 3;
    const float *prepared = nullptr;
    const int8_t *bp[NG], *sp[NG];
    const float *fe[NG], *fo[NG];   // Q5_1: per-block sums of the even / odd activation row of each column group
    float xs[2 * NG];   // this warp's scale of each activation row
    Accum<NG> acc;
    AccumSingle acs;
    accum_zero(acc);
    acs.f[0] = acs.f[1] = acs.m[0] = acs.m[1] = acs.m[2] = acs.m[3] = 0.0f;
    int tile_it = 0;
    // With stacked tiles warp w holds unit w % units of sub-tile w / units of every stage; otherwise units
    // w, w + 8, ... of the stage (a stage holds at most 8 units unless it is one whole tile).
    const int my_sub = STACK ? wid / p.units : 0;
    const int my_unit = STACK ? wid - my_sub * p.units : wid;
    const bool stacked_idle = STACK && my_sub >= tps;
    const uint32_t lane_off = (uint32_t)(kTileRows * my_sub + g) * p.row_stride;
    if (!stacked_idle) {
        planes += my_sub * plane_bytes<WT>(p.n_in, p.rows);
        chunk_sum += my_sub * chunk_sum_bytes<WT>(p.n_in, p.rows);
    }
    // single-row form: column g = limb g/2 of the low (g even) or high (g odd) chunk of a group
    const int8_t *bq = planes + (g < 6 ? (g >> 1) * plane_stride(p.n_in) + (WT == KRK_CUDA_Q4_0 ? 16 : 32) * (g & 1) : 0);
    const int8_t *sq = chunk_sum + (g & 3) * (p.n_in >> 5);
    BFrag held[2];

    // The same walk as walk() above, written flat: per stage a consumer warp only needs the ring
    // slot and its K units, not which matrix or rows the tile belongs to.
    const int cta = (int)blockIdx.x;
    const int g0 = cta * tv.gran_q + min(cta, tv.gran_r);
    const int g1 = g0 + tv.gran_q + (cta < tv.gran_r ? 1 : 0);
    const int n_chunks = p.whole_tiles ? 1 : (p.units + kConsumerWarps - 1) / kConsumerWarps;
    const uint32_t full0 = smem_u32(&sm->full[0]), empty0 = smem_u32(&sm->empty[0]);
    int slot = 0;
    uint32_t phase = 0;
    for (int e = 0; e < tv.n_entries; e++) {
        const int lo = max(g0, tv.gran_begin[e]), hi = min(g1, tv.gran_begin[e + 1]);
        if (lo >= hi) continue;
        const int m = e * p.step;
        const int r0 = (lo - tv.gran_begin[e]) * p.gran;
        const int r1 = min((int)tv.mat[m].n_out, (hi - tv.gran_begin[e]) * p.gran);
        if (tv.mat[m].x != prepared) {
            // x may be the output of the kernel before this one (and y its input): wait for that grid to
            // complete. Weights are never written by a kernel in flight, so the producer warp does not wait.
            if (prepared == nullptr) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                if (p.tune & 2) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            }
            prepared = tv.mat[m].x;
#pragma unroll
            for (int r = 0; r < 2 * NG; r++)
                // (stacked tiles: every sub-tile prepares its own copy)
                xs[r] = r < p.rows ? prepare_x_row<WT>(prepared + (size_t)r * p.n_in, p,
                                                       planes + (size_t)(r * 3) * plane_stride(p.n_in),
                                                       chunk_sum + (size_t)(r * 4) * (p.n_in >> kSumShift<WT>),
                                                       stacked_idle ? kConsumerWarps : my_unit, lane)
                                   : 0.0f;
            __syncwarp();
            if (!SINGLE) lane_planes<NG>(planes, chunk_sum, p.n_in, p.n_in >> kSumShift<WT>, p.rows, g, bp, sp);
            if (WT == KRK_CUDA_Q5_1) {
#pragma unroll
                for (int mg = 0; mg < NG; mg++) {   // per-block sums of the group's even and odd activation rows
                    fe[mg] = reinterpret_cast<const float *>(chunk_sum) + (size_t)min(2 * mg, p.rows - 1) * (p.n_in >> 5);
                    fo[mg] = reinterpret_cast<const float *>(chunk_sum) + (size_t)min(2 * mg + 1, p.rows - 1) * (p.n_in >> 5);
                }
            }
            if (SINGLE == 2 && !stacked_idle) {
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int u = my_unit + j * kConsumerWarps;
                    if (u < p.units) held[j] = load_bfrag(bq + u * F::unit_values, sq + ((u * F::unit_values) >> 5), t);
                }
            }
        }
        const int stage_rows = kTileRows * tps;
        const int n_tiles = ((r1 - r0 + stage_rows - 1) / stage_rows) * p.step;
        for (int tile = 0; tile < n_tiles; tile++) {
            // ragged rows: how far this lane's two rows sit into their slots of a stage
            uint32_t ragA = 0, ragB = 0;
            if (RAG || (WT == KRK_CUDA_Q2_K && p.ragged)) {
                const int row = r0 + (tile / p.step) * stage_rows + kTileRows * my_sub + g;
                const uintptr_t base = reinterpret_cast<uintptr_t>(tv.mat[m + tile % p.step].w);
                ragA = (uint32_t)((base + (size_t)row * p.row_bytes) & 15);
                ragB = (uint32_t)((base + (size_t)(row + 8) * p.row_bytes) & 15);
            }
            // one stage of the tile: `bf` are the warp's held B fragments for it (SINGLE == 2), else unused
            auto stage = [&](const int ck, const BFrag &bf) {
                wait_phase(full0 + 8 * slot, phase, gave_up, p.status);
                const int stage_units = p.whole_tiles ? p.units : min(kConsumerWarps, p.units - ck * kConsumerWarps);
                if (!stacked_idle) {
                    const uint8_t *tile0 = stages + (size_t)slot * p.stage_bytes + lane_off;
                    for (int su = my_unit; su < stage_units; su += kConsumerWarps) {
                        const uint8_t *rowA = tile0 + (size_t)su * p.unit_stride + ragA;
                        const uint8_t *rowB = tile0 + (size_t)su * p.unit_stride + (size_t)8 * p.row_stride + ragB;
                        const int unit = ck * kConsumerWarps + su;
                        const int kbase = unit * F::unit_values;
                        if (WT == KRK_CUDA_Q4_0 && !SINGLE) {
                            unit_q4_0_rows<NG>(rowA, rowB, kbase, bp, t, acc);
                        } else if (WT == KRK_CUDA_Q4_0) {
                            unit_q4_0(rowA, rowB, bq + kbase, reinterpret_cast<const float *>(chunk_sum) + (kbase >> 5), t, acs);
                        } else if (SINGLE == 2) {
                            unit_q4_k_single(rowA, rowB, bf, t, acs);
                        } else if (SINGLE == 1) {
                            unit_q4_k_single(rowA, rowB, load_bfrag(bq + kbase, sq + (kbase >> 5), t), t, acs);
                        } else if (WT == KRK_CUDA_Q4_K || WT == KRK_CUDA_Q5_K) {
                            unit_q4_k<NG, WT == KRK_CUDA_Q5_K>(rowA, rowB, kbase, bp, sp, t, acc);
                        } else if (WT == KRK_CUDA_Q8_0) {
                            unit_q8_0<NG>(rowA, rowB, kbase, bp, t, acc);
                        } else if (WT == KRK_CUDA_Q5_0) {
                            unit_q5_0<NG>(rowA, rowB, kbase, bp, t, acc);
                        } else if (WT == KRK_CUDA_IQ4_NL) {
                            unit_iq4_nl<NG>(rowA, rowB, kbase, bp, t, acc);
                        } else if (WT == KRK_CUDA_Q2_K) {
                            unit_q2_k<NG>(rowA, rowB, kbase, bp, sp, t, acc);
                        } else if (WT == KRK_CUDA_Q3_K) {
                            if (RAG) unit_q3_k<NG, 2>(rowA, rowB, kbase, bp, t, acc);
                            else if (unit & 1) unit_q3_k<NG, 1>(rowA, rowB, kbase, bp, t, acc);
                            else unit_q3_k<NG, 0>(rowA, rowB, kbase, bp, t, acc);
                        } else if (WT == KRK_CUDA_Q5_1) {
                            unit_q5_1<NG>(rowA, rowB, kbase, bp, fe, fo, t, acc);
                        } else {
                            if (RAG) unit_q6_k<NG, 2>(rowA, rowB, kbase, bp, t, acc);
                            else if (unit & 1) unit_q6_k<NG, 1>(rowA, rowB, kbase, bp, t, acc);
                            else unit_q6_k<NG, 0>(rowA, rowB, kbase, bp, t, acc);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * slot);
                if (++slot == p.n_stages) {
                    slot = 0;
                    phase ^= 1;
                }
            };
            if (SINGLE == 2) {   // at most two stages per tile, each with its own registers
                stage(0, held[0]);
                if (n_chunks > 1) stage(1, held[1]);
            } else {
                for (int ck = 0; ck < n_chunks; ck++) stage(ck, held[0]);
            }
            {
             // ---- end of the tile: the four lanes of a row group add their weighted shares, lane t = 0 leaves them ----
             constexpr int kSlots = red_slots(NG);
             const int rslot = tile_it % kSlots;
             const uint32_t rphase = (tile_it / kSlots) & 1;
             tile_it++;
             if (wid >= n_warps) continue;
             // min columns: limb c%4 (weights 2^24, 2^16, 2^8, 1) of activation row c/4
             const float me0 = t == 0 ? 16777216.0f : (t == 1 ? 256.0f : 0.0f), me1 = t == 0 ? 65536.0f : (t == 1 ? 1.0f : 0.0f);
             const float mo0 = t == 2 ? 16777216.0f : (t == 3 ? 256.0f : 0.0f), mo1 = t == 2 ? 65536.0f : (t == 3 ? 1.0f : 0.0f);
             float4 o[NG];
             if (SINGLE) {
                 // lane t holds limb t (weights 65536, 256, 1) of rows g and g+8, times 16
                 // (Q4_0: lane t = 3 holds d * sum of X per block, the -8 of every quant)
                 const float wl = t == 0 ? 4096.0f : (t == 1 ? 16.0f : (t == 2 ? 0.0625f : (WT == KRK_CUDA_Q4_0 ? -8.0f : 0.0f)));
                 o[0].x = (wl * acs.f[0] - fmaf(me0, acs.m[0], me1 * acs.m[1])) * xs[0];
                 o[0].z = (wl * acs.f[1] - fmaf(me0, acs.m[2], me1 * acs.m[3])) * xs[0];
                 o[0].y = o[0].w = 0.0f;
                 acs.f[0] = acs.f[1] = acs.m[0] = acs.m[1] = acs.m[2] = acs.m[3] = 0.0f;
             } else {
                 // Column c of a group carries limb c%3 (weights 65536, 256, 1) of activation row c/3; this lane
                 // holds columns 2t and 2t+1, so its accumulators enter the even activation row with (we0, we1)
                 // and the odd one with (wo0, wo1). The Q4_K min term is already a per-lane partial sum.
                 const float we0 = t == 0 ? 65536.0f : (t == 1 ? 1.0f : 0.0f), we1 = t == 0 ? 256.0f : 0.0f;
                 const float wo0 = t == 2 ? 256.0f : 0.0f, wo1 = t == 1 ? 65536.0f : (t == 2 ? 1.0f : 0.0f);
#pragma unroll
                 for (int mg = 0; mg < NG; mg++) {
                     if (NG == 4 && mg == 3) {
                         // activation rows 6 and 7 rode in columns 6 and 7 (lane t = 3) of groups 0..2, limb mg in group mg
                         const float w0 = t == 3 ? 65536.0f : 0.0f, w1 = t == 3 ? 256.0f : 0.0f, w2 = t == 3 ? 1.0f : 0.0f;
                         o[mg].x = fmaf(w0, acc.f[0][0], fmaf(w1, acc.f[1][0], w2 * acc.f[2][0]));
                         o[mg].y = fmaf(w0, acc.f[0][1], fmaf(w1, acc.f[1][1], w2 * acc.f[2][1]));
                         o[mg].z = fmaf(w0, acc.f[0][2], fmaf(w1, acc.f[1][2], w2 * acc.f[2][2]));
                         o[mg].w = fmaf(w0, acc.f[0][3], fmaf(w1, acc.f[1][3], w2 * acc.f[2][3]));
                     } else {
                         o[mg].x = fmaf(we0, acc.f[mg][0], we1 * acc.f[mg][1]);   // row g,   even activation row
                         o[mg].y = fmaf(wo0, acc.f[mg][0], wo1 * acc.f[mg][1]);   // row g,   odd
                         o[mg].z = fmaf(we0, acc.f[mg][2], we1 * acc.f[mg][3]);   // row g+8, even
                         o[mg].w = fmaf(wo0, acc.f[mg][2], wo1 * acc.f[mg][3]);   // row g+8, odd
                     }
                     if (WT == KRK_CUDA_Q4_K || WT == KRK_CUDA_Q5_K || WT == KRK_CUDA_Q2_K) {
                         o[mg].x -= fmaf(me0, acc.m[mg][0], me1 * acc.m[mg][1]);
                         o[mg].y -= fmaf(mo0, acc.m[mg][0], mo1 * acc.m[mg][1]);
                         o[mg].z -= fmaf(me0, acc.m[mg][2], me1 * acc.m[mg][3]);
                         o[mg].w -= fmaf(mo0, acc.m[mg][2], mo1 * acc.m[mg][3]);
                     }
                     o[mg].x *= xs[2 * mg];
                     o[mg].y *= xs[2 * mg + 1];
                     o[mg].z *= xs[2 * mg];
                     o[mg].w *= xs[2 * mg + 1];
                 }
                 accum_zero(acc);
             }
#pragma unroll
             for (int mg = 0; mg < NG; mg++) {
#pragma unroll
                 for (int d = 1; d <= 2; d <<= 1) {   // (t0 + t1) + (t2 + t3): a fixed order
                     o[mg].x += __shfl_xor_sync(0xFFFFFFFFu, o[mg].x, d);
                     o[mg].z += __shfl_xor_sync(0xFFFFFFFFu, o[mg].z, d);
                     if (!SINGLE) {
                         o[mg].y += __shfl_xor_sync(0xFFFFFFFFu, o[mg].y, d);
                         o[mg].w += __shfl_xor_sync(0xFFFFFFFFu, o[mg].w, d);
                     }
                 }
             }
             wait_phase(smem_u32(&sm->red_empty[rslot]), rphase ^ 1, gave_up, p.status);
             if (t == 0) {
#pragma unroll
                 for (int mg = 0; mg < NG; mg++) sm->red[rslot][wid][mg][g] = o[mg];
             }
             __syncwarp();
             if (lane == 0) mbar_arrive(smem_u32(&sm->red_full[rslot]));
            }
        }
    }
}

template <int WT, int NG, bool STACK, int SINGLE, bool RAG = false>
int launch_one(const StreamParams &p, int grid, size_t smem, cudaStream_t st) {
    static bool configured[64] = {};   // per instantiation and device: the opt-in is sticky
    auto kernel = gemv_stream_kernel<WT, NG, STACK, SINGLE, RAG>;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemWhole);
        // all of the SM's configurable memory as shared memory, so that two CTAs fit
        if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        if (e != cudaSuccess) {
            note_cuda_error(e);
            return KRK_CUDA_ELAUNCH;
        }
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p);
    note_launch(1, KRK_CUDA_FAMILY_GEMV_STREAM);
    if (e != cudaSuccess) {
        note_cuda_error(e);
        (void)cudaGetLastError();
        return KRK_CUDA_ELAUNCH;
    }
    return KRK_CUDA_OK;
}

// Fills the fields that depend only on the format, the width and the activation row count.
// Returns false when the streaming kernel does not address the shape.
template <int WT>
bool setup_format(StreamParams &p, int64_t n_in, int rows, int silu_pair, size_t *smem_out, bool want_tma = false) {
    using F = Fmt<WT>;
    if (n_in % 256 != 0 || n_in > (1 << 20) || rows < 1 || rows > KRK_CUDA_MAX_ROWS) return false;
    p.n_in = (int)n_in;
    p.units = (int)(n_in / F::unit_values);
    p.row_bytes = (int)row_bytes(WT, n_in);
    p.rows = rows;
    p.accumulate = 0;
    p.step = silu_pair ? 2 : 1;
    p.whole_tiles = 0;
    p.ragged = 0;
    p.gran = 1;
    p.dev_table = nullptr;
    p.n_peers = 0;
    p.my_rank = p.epoch = 0;
    p.peer_row_stride = p.peer_offset = 0;
    if (WT == KRK_CUDA_Q6_K && (n_in % 2048) != 0) {
        // 210-byte blocks: rows are 16-byte multiples only for K % 2048 == 0. Otherwise whole 16-row
        // tiles are copied contiguously (needs 4-byte-multiple rows and the tile in one stage), or, for longer
        // or odd rows (K = 11008: 9030 bytes), row by row from the 16-byte boundary below each row.
        if ((p.row_bytes & 3) == 0 && p.units <= 2 * kConsumerWarps) {
            p.whole_tiles = 1;
            p.gran = 8;
        } else {
            p.ragged = 1;
        }
    }
    // Q2_K rows are 16-byte multiples for K % 1024 == 0, Q3_K rows for K % 2048 == 0
    if ((WT == KRK_CUDA_Q2_K || WT == KRK_CUDA_Q3_K) && (p.row_bytes & 15) != 0) p.ragged = 1;
    const int ku_max = p.whole_tiles ? p.units : (p.units < kConsumerWarps ? p.units : kConsumerWarps);
    p.tps = kConsumerWarps / p.units;   // 0 when a tile has more units than there are consumer warps
    p.tps = p.tps < 1 ? 1 : (p.tps > kMaxStack ? kMaxStack : p.tps);
    p.use_tma = 0;
    p.box_bytes = 0;
    static const int tune = [] {
        const char *e = std::getenv("KRK_CUDA_GEMV_TUNE");
        return e ? std::atoi(e) : 0;
    }();
    p.tune = tune;
    p.unit_stride = F::unit_bytes;
    p.tma_unit_div = 1;
    if (want_tma && F::tma == 1 && !p.whole_tiles) {
        // a stage is one tensor copy: [units of the stage][rows of the stage][unit_bytes]. The 144-byte
        // pitch of a Q4_K unit puts the eight rows of a fragment load 16 bytes apart in the banks.
        p.use_tma = 1;
        p.row_stride = F::unit_bytes;
        p.unit_stride = kTileRows * p.tps * F::unit_bytes;
        p.box_bytes = ku_max * p.unit_stride;
        p.stage_bytes = align_up(p.box_bytes, 128);
        p.gran = kTileRows * p.tps;   // a copy brings whole tiles: CTAs split the rows at tile boundaries, so no row is fetched twice
    } else if (want_tma && F::tma == 2 && !p.whole_tiles && ku_max == kConsumerWarps && p.units % kConsumerWarps == 0) {
        // a stage is one tensor copy of eight units of each row: [row][8 units], pitch 8 * unit_bytes (1680 for
        // Q6_K: the rows of a fragment load again lie 16 bytes apart in the banks)
        p.use_tma = 2;
        p.tma_unit_div = kConsumerWarps;
        p.row_stride = ku_max * F::unit_bytes;
        p.box_bytes = kTileRows * p.tps * p.row_stride;
        p.stage_bytes = align_up(p.box_bytes, 128);
        p.gran = kTileRows * p.tps;
    } else if (p.whole_tiles) {
        p.row_stride = p.row_bytes;
        p.stage_bytes = align_up(kTileRows * p.tps * p.row_bytes, 128);
    } else {
        // (ragged rows: up to 15 bytes before and 15 after the row's own, and a word of slack for the loads that
        // glue a value from two words)
        const int raw = ku_max * F::unit_bytes + (p.ragged ? 48 : 0);
        p.row_stride = raw + ((F::stride_mod - raw % 128) + 128) % 128;
        p.stage_bytes = align_up(kTileRows * p.tps * p.row_stride, 128);
    }
    const int smem_struct = rows <= 2 ? (int)sizeof(Smem<1>) : rows <= 4 ? (int)sizeof(Smem<2>) : (int)sizeof(Smem<4>);
    const int fixed = align_up(smem_struct, 128) + p.tps * (plane_bytes<WT>(p.n_in, rows) + chunk_sum_bytes<WT>(p.n_in, rows));
    // Depth of the ring: as many stages as fit beside the prepared activation in half an SM, at most
    // kMaxStages. Wide activations (large K) leave too little of a half, and the forms compiled for one CTA
    // per SM (more registers; see kTwoPerSm) take the whole SM.
    const bool halves = rows <= 2 || (rows <= 4 && kTwoPerSm<WT, 2>);
    int max_fit = halves ? (kSmemLimit - fixed) / p.stage_bytes : 0;
    if (max_fit < 3) max_fit = (kSmemWhole - fixed) / p.stage_bytes;
    p.n_stages = max_fit < kMaxStages ? max_fit : kMaxStages;
    if (p.n_stages < 2) return false;
    *smem_out = (size_t)fixed + (size_t)p.n_stages * p.stage_bytes;
    return true;
}

template <int WT>
int launch_rows(const StreamParams &p, int grid, size_t smem, cudaStream_t st) {
    constexpr bool kQ4K = WT == KRK_CUDA_Q4_K;
    if constexpr (WT == KRK_CUDA_Q4_0) {
        if (p.rows == 1) return p.tps > 1 ? launch_one<WT, 1, true, 1>(p, grid, smem, st) : launch_one<WT, 1, false, 1>(p, grid, smem, st);
        if (p.rows <= 2) return p.tps > 1 ? launch_one<WT, 1, true, 0>(p, grid, smem, st) : launch_one<WT, 1, false, 0>(p, grid, smem, st);
        if (p.rows <= 4) return p.tps > 1 ? launch_one<WT, 2, true, 0>(p, grid, smem, st) : launch_one<WT, 2, false, 0>(p, grid, smem, st);
        return p.tps > 1 ? launch_one<WT, 4, true, 0>(p, grid, smem, st) : launch_one<WT, 4, false, 0>(p, grid, smem, st);
    } else {
        if constexpr (WT == KRK_CUDA_Q6_K || WT == KRK_CUDA_Q3_K) {
            if (p.ragged) {
                if (p.tps > 1) {
                    if (p.rows <= 2) return launch_one<WT, 1, true, 0, true>(p, grid, smem, st);
                    if (p.rows <= 4) return launch_one<WT, 2, true, 0, true>(p, grid, smem, st);
                    return launch_one<WT, 4, true, 0, true>(p, grid, smem, st);
                }
                if (p.rows <= 2) return launch_one<WT, 1, false, 0, true>(p, grid, smem, st);
                if (p.rows <= 4) return launch_one<WT, 2, false, 0, true>(p, grid, smem, st);
                return launch_one<WT, 4, false, 0, true>(p, grid, smem, st);
            }
        }
        if (p.tps > 1) {
            if (kQ4K && p.rows == 1) return launch_one<WT, 1, true, kQ4K ? 2 : 0>(p, grid, smem, st);
            if (p.rows <= 2) return launch_one<WT, 1, true, 0>(p, grid, smem, st);
            if (p.rows <= 4) return launch_one<WT, 2, true, 0>(p, grid, smem, st);
            return launch_one<WT, 4, true, 0>(p, grid, smem, st);
        }
        if (kQ4K && p.rows == 1 && !p.whole_tiles && p.units <= 2 * kConsumerWarps) return launch_one<WT, 1, false, kQ4K ? 2 : 0>(p, grid, smem, st);
        if (kQ4K && p.rows == 1) return launch_one<WT, 1, false, kQ4K ? 1 : 0>(p, grid, smem, st);
        if (p.rows <= 2) return launch_one<WT, 1, false, 0>(p, grid, smem, st);
        if (p.rows <= 4) return launch_one<WT, 2, false, 0>(p, grid, smem, st);
        return launch_one<WT, 4, false, 0>(p, grid, smem, st);
    }
}

// CTAs of one launch per SM. 2 (default): both halves of an SM work on this launch (16 consumer warps per SM:
// 0.80-0.83 of the copy bandwidth on large Q4_K / Q8_0 matrices against 0.5-0.7 with one). 1
// (KRK_CUDA_GEMV_CTAS_PER_SM=1): the other half is left to the next launch in the stream, which becomes
// resident early, sets itself up and fills its ring while this one streams; measured on the layer-sized
// matrices of a decode step the slower streaming of eight warps costs more than the overlap saves.
// The forms compiled for one CTA per SM (kTwoPerSm) get one whatever their shared memory: a grid of two per
// SM would run as two waves and prepare the activation twice.
template <int WT>
int ctas_per_sm(size_t smem, int rows) {
    static const int want = [] {
        const char *e = std::getenv("KRK_CUDA_GEMV_CTAS_PER_SM");
        const int v = e ? std::atoi(e) : 0;
        return v == 1 ? 1 : 2;
    }();
    const bool halves = rows <= 2 || (rows <= 4 && kTwoPerSm<WT, 2>);
    return halves && smem <= (size_t)kSmemLimit ? want : 1;
}

// Tensor maps are encoded on the host (a driver call of a microsecond or two) and kept per (matrix, box):
// weights stay where they were uploaded, so a decode loop encodes each matrix once.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct MapKey {
    const void *w;
    int64_t n_out;
    int row_bytes, unit_bytes, box_rows, box_units;
    bool operator==(const MapKey &o) const {
        return w == o.w && n_out == o.n_out && row_bytes == o.row_bytes && unit_bytes == o.unit_bytes &&
               box_rows == o.box_rows && box_units == o.box_units;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey &k) const {
        size_t h = reinterpret_cast<size_t>(k.w) * 0x9E3779B97F4A7C15ull;
        h ^= (size_t)k.n_out * 0xC2B2AE3D27D4EB4Full + (size_t)k.row_bytes * 31 + (size_t)k.box_rows * 7 + (size_t)k.box_units;
        return h;
    }
};
CUtensorMapL2promotion l2_promotion() {
    static const int v = [] {
        const char *e = std::getenv("KRK_CUDA_GEMV_L2PROMO");
        return e ? std::atoi(e) : 3;
    }();
    return v == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : v == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
           : v == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
}
bool weight_map(CUtensorMap *out, const uint8_t *w, int64_t n_out, int row_bytes, int unit_bytes, int box_rows, int box_units,
                int mode) {
    static EncodeTiledFn encode = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    if (!encode) return false;
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{w, n_out, row_bytes, unit_bytes, box_rows, mode == 2 ? -box_units : box_units};
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    // mode 1: {unit bytes, rows, units of a row} in bytes; mode 2: {box_units units as 64-bit elements, rows, groups of
    // box_units units of a row}
    const int inner_bytes = mode == 2 ? box_units * unit_bytes : unit_bytes;
    if (mode == 2 && (inner_bytes % 16 != 0 || inner_bytes / 8 > 256 || row_bytes % inner_bytes != 0)) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)(mode == 2 ? inner_bytes / 8 : inner_bytes), (cuuint64_t)n_out,
                                (cuuint64_t)(row_bytes / inner_bytes)};
    const cuuint64_t strides[2] = {(cuuint64_t)row_bytes, (cuuint64_t)inner_bytes};
    const cuuint32_t box[3] = {(cuuint32_t)dims[0], (cuuint32_t)box_rows, (cuuint32_t)(mode == 2 ? 1 : box_units)};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUtensorMap m;
    if (encode(&m, mode == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT64 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t *>(w), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, l2_promotion(),
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 65536) cache.clear();   // bounded: a host that keeps re-uploading weights starts over
    cache.emplace(key, m);
    *out = m;
    return true;
}

// Fills p.wmap for the first n matrices of p.mat; on failure the launch falls back to row copies.
template <int WT>
bool encode_maps(StreamParams &p, int n) {
    using F = Fmt<WT>;
    const int ku_max = p.units < kConsumerWarps ? p.units : kConsumerWarps;
    for (int m = 0; m < n; m++) {
        if (p.mat[m].n_out <= 0) continue;
        if ((reinterpret_cast<uintptr_t>(p.mat[m].w) & 15) != 0) return false;
        if (!weight_map(&p.wmap[m], p.mat[m].w, p.mat[m].n_out, p.row_bytes, F::unit_bytes, kTileRows * p.tps, ku_max, p.use_tma)) return false;
    }
    return true;
}

// setup_format with the tensor-copy layout where the format and the matrices allow it (the maps are encoded here),
// else with per-row copies. False when the streaming kernel does not address the shape.
template <int WT>
bool setup_launch(StreamParams &p, const GemvMat *mats, int n_mat, int64_t n_in, int rows, int silu_pair, size_t *smem) {
    static const bool no_tma = std::getenv("KRK_CUDA_GEMV_NO_TMA") != nullptr;
    bool tma = Fmt<WT>::tma != 0 && !no_tma;
    if (tma) {
        if (!setup_format<WT>(p, n_in, rows, silu_pair, smem, true)) return false;
        if (p.use_tma) {
            for (int m = 0; m < n_mat; m++) p.mat[m] = mats[m];
            if (!encode_maps<WT>(p, n_mat)) tma = false;   // a map cannot be encoded: set up again for row copies
        }
    }
    return tma || setup_format<WT>(p, n_in, rows, silu_pair, smem);
}

template <int WT>
int launch_fmt(const GemvMat *mats, int n_mat, int64_t n_in, int rows, int accumulate, int silu_pair, cudaStream_t st) {
    StreamParams p;
    size_t smem = 0;
    if (!setup_launch<WT>(p, mats, n_mat, n_in, rows, silu_pair, &smem)) return 0;
    p.accumulate = accumulate;
    p.n_entries = 0;
    int total = 0;
    for (int m = 0; m < n_mat; m += p.step) {
        if (mats[m].n_out > (1 << 30)) return 0;
        for (int j = 0; j < p.step; j++) p.mat[p.n_entries * p.step + j] = mats[m + j];
        p.gran_begin[p.n_entries] = total;
        total += (int)((mats[m].n_out + p.gran - 1) / p.gran);
        p.n_entries++;
    }
    p.gran_begin[p.n_entries] = total;
    p.total_gran = total;
    if (total == 0) return 1;
    p.status = device_status_word();
    if (!p.status) return KRK_CUDA_EDEVICE;
    const int sms = sm_count() * ctas_per_sm<WT>(smem, p.rows);
    const int grid = total < sms ? total : sms;
    p.gran_q = total / grid;
    p.gran_r = total % grid;
    const int rc = launch_rows<WT>(p, grid, smem, st);
    return rc == KRK_CUDA_OK ? 1 : rc;
}

template <int WT>
int gran_fmt(int64_t n_in, bool banks) {
    StreamParams p;
    size_t smem = 0;
    static const bool no_tma = std::getenv("KRK_CUDA_GEMV_NO_TMA") != nullptr;
    if (banks && Fmt<WT>::tma == 1 && !no_tma && setup_format<WT>(p, n_in, 1, 0, &smem, true) && p.use_tma == 1) return p.gran;
    return setup_format<WT>(p, n_in, 1, 0, &smem) ? p.gran : 0;
}

template <int WT>
int launch_table_fmt(const StreamTable *table, int64_t n_in, int silu_pair, const StreamBanks *banks, cudaStream_t st) {
    StreamParams p;
    size_t smem = 0;
    // With the banks known, a stage arrives as one tensor copy out of the bank's map (the table must then have been
    // built with the granule of stream_gran(..., true): rows split at tile boundaries).
    static const bool no_tma = std::getenv("KRK_CUDA_GEMV_NO_TMA") != nullptr;
    bool tma = false;
    if (banks && Fmt<WT>::tma == 1 && !no_tma && setup_format<WT>(p, n_in, 1, silu_pair, &smem, true) && p.use_tma == 1) {
        tma = true;
        const int ku_max = p.units < kConsumerWarps ? p.units : kConsumerWarps;
        for (int b = 0; b < p.step && tma; b++) {
            p.bank_base[b] = banks->base[b];
            tma = banks->base[b] && (reinterpret_cast<uintptr_t>(banks->base[b]) & 15) == 0 && banks->rows > 0 &&
                  weight_map(&p.wmap[b], banks->base[b], banks->rows, p.row_bytes, Fmt<WT>::unit_bytes, kTileRows * p.tps, ku_max, 1);
        }
    }
    if (!tma && !setup_format<WT>(p, n_in, 1, silu_pair, &smem)) return 0;
    // the table was built with this granule whichever way the stages arrive (row copies take any granule)
    if (banks) p.gran = gran_fmt<WT>(n_in, true);
    p.n_entries = 0;
    p.total_gran = 0;
    p.gran_q = p.gran_r = 0;
    p.dev_table = table;
    p.status = device_status_word();
    if (!p.status) return KRK_CUDA_EDEVICE;
    const int rc = launch_rows<WT>(p, sm_count() * ctas_per_sm<WT>(smem, p.rows), smem, st);
    return rc == KRK_CUDA_OK ? 1 : rc;
}

template <int WT>
int launch_peers_fmt(const GemvMat &mat, int64_t n_in, int rows, const PeerScatter &ps, cudaStream_t st) {
    StreamParams p;
    size_t smem = 0;
    if (mat.n_out > (1 << 30) || mat.n_out <= 0) return 0;
    if (!setup_launch<WT>(p, &mat, 1, n_in, rows, 0, &smem)) return 0;
    p.mat[0] = mat;
    p.n_entries = 1;
    p.gran_begin[0] = 0;
    const int total = (int)((mat.n_out + p.gran - 1) / p.gran);
    p.gran_begin[1] = total;
    p.total_gran = total;
    p.status = device_status_word();
    if (!p.status) return KRK_CUDA_EDEVICE;
    p.n_peers = ps.n_peers;
    for (int q = 0; q < ps.n_peers; q++) {
        p.peer_y[q] = ps.y[q];
        p.peer_flag[q] = ps.flag[q];
    }
    p.my_rank = ps.my_rank;
    p.epoch = ps.epoch;
    p.wait_peers = ps.wait_peers;
    p.peer_row_stride = ps.row_stride;
    p.peer_offset = ps.offset;
    const int sms = sm_count() * ctas_per_sm<WT>(smem, p.rows);
    const int grid = total < sms ? total : sms;
    p.gran_q = total / grid;
    p.gran_r = total % grid;
    const int rc = launch_rows<WT>(p, grid, smem, st);
    return rc == KRK_CUDA_OK ? 1 : rc;
}

// One warp: lane q waits (bounded) until flag[q] has reached `epoch`, i.e. until peer q has stored its
// slice of the row into this GPU's buffer. A wait that gives up raises the device status word.
__global__ void __launch_bounds__(32) flag_wait_kernel(const int *flags, int n, int epoch, int *status) {
    const int q = threadIdx.x;
    if (q < n) {
        const long long t0 = clock64();
        while (*reinterpret_cast<const volatile int *>(flags + q) < epoch) {
            __nanosleep(200);
            if (clock64() - t0 > kWaitCycles) {
                atomicExch(status, KRK_CUDA_ETIMEOUT);
                break;
            }
        }
    }
    __threadfence_system();
}

} // namespace

int launch_gemv_stream(const GemvMat *mats, int n_mat, int64_t n_in, int rows, int accumulate, int silu_pair,
                       cudaStream_t st) {
    if (n_mat < 1 || rows < 1 || rows > KRK_CUDA_MAX_ROWS) return 0;
    const int wt = mats[0].wt;
    for (int m = 1; m < n_mat; m++)
        if (mats[m].wt != wt) return 0;
    switch (wt) {
    case KRK_CUDA_Q4_K: return launch_fmt<KRK_CUDA_Q4_K>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q6_K: return launch_fmt<KRK_CUDA_Q6_K>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q8_0: return launch_fmt<KRK_CUDA_Q8_0>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q4_0: return launch_fmt<KRK_CUDA_Q4_0>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q5_K: return launch_fmt<KRK_CUDA_Q5_K>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q2_K: return launch_fmt<KRK_CUDA_Q2_K>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q3_K: return launch_fmt<KRK_CUDA_Q3_K>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_IQ4_NL: return launch_fmt<KRK_CUDA_IQ4_NL>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q5_0: return launch_fmt<KRK_CUDA_Q5_0>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    case KRK_CUDA_Q5_1: return launch_fmt<KRK_CUDA_Q5_1>(mats, n_mat, n_in, rows, accumulate, silu_pair, st);
    default: return 0;   // the other formats take the shape-agnostic kernel
    }
}

int launch_gemv_stream_table(const StreamTable *table, int wt, int64_t n_in, int silu_pair, const StreamBanks *banks,
                             cudaStream_t st) {
    switch (wt) {
    case KRK_CUDA_Q4_K: return launch_table_fmt<KRK_CUDA_Q4_K>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q6_K: return launch_table_fmt<KRK_CUDA_Q6_K>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q8_0: return launch_table_fmt<KRK_CUDA_Q8_0>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q4_0: return launch_table_fmt<KRK_CUDA_Q4_0>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q5_K: return launch_table_fmt<KRK_CUDA_Q5_K>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q2_K: return launch_table_fmt<KRK_CUDA_Q2_K>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q3_K: return launch_table_fmt<KRK_CUDA_Q3_K>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_IQ4_NL: return launch_table_fmt<KRK_CUDA_IQ4_NL>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q5_0: return launch_table_fmt<KRK_CUDA_Q5_0>(table, n_in, silu_pair, banks, st);
    case KRK_CUDA_Q5_1: return launch_table_fmt<KRK_CUDA_Q5_1>(table, n_in, silu_pair, banks, st);
    default: return 0;
    }
}

int launch_gemv_stream_peers(const GemvMat &mat, int64_t n_in, int rows, const PeerScatter &ps, cudaStream_t st) {
    switch (mat.wt) {
    case KRK_CUDA_Q4_K: return launch_peers_fmt<KRK_CUDA_Q4_K>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q6_K: return launch_peers_fmt<KRK_CUDA_Q6_K>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q8_0: return launch_peers_fmt<KRK_CUDA_Q8_0>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q4_0: return launch_peers_fmt<KRK_CUDA_Q4_0>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q5_K: return launch_peers_fmt<KRK_CUDA_Q5_K>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q2_K: return launch_peers_fmt<KRK_CUDA_Q2_K>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q3_K: return launch_peers_fmt<KRK_CUDA_Q3_K>(mat, n_in, rows, ps, st);
    case KRK_CUDA_IQ4_NL: return launch_peers_fmt<KRK_CUDA_IQ4_NL>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q5_0: return launch_peers_fmt<KRK_CUDA_Q5_0>(mat, n_in, rows, ps, st);
    case KRK_CUDA_Q5_1: return launch_peers_fmt<KRK_CUDA_Q5_1>(mat, n_in, rows, ps, st);
    default: return 0;
    }
}

int launch_flag_wait(const int *flags, int n, int epoch, cudaStream_t st) {
    int *status = device_status_word();
    if (!status) return KRK_CUDA_EDEVICE;
    flag_wait_kernel<<<1, 32, 0, st>>>(flags, n, epoch, status);
    note_launch();
    return check_launch();
}

int stream_gran(int wt, int64_t n_in, bool banks) {
    switch (wt) {
    case KRK_CUDA_Q4_K: return gran_fmt<KRK_CUDA_Q4_K>(n_in, banks);
    case KRK_CUDA_Q6_K: return gran_fmt<KRK_CUDA_Q6_K>(n_in, banks);
    case KRK_CUDA_Q8_0: return gran_fmt<KRK_CUDA_Q8_0>(n_in, banks);
    case KRK_CUDA_Q4_0: return gran_fmt<KRK_CUDA_Q4_0>(n_in, banks);
    case KRK_CUDA_Q5_K: return gran_fmt<KRK_CUDA_Q5_K>(n_in, banks);
    case KRK_CUDA_Q2_K: return gran_fmt<KRK_CUDA_Q2_K>(n_in, banks);
    case KRK_CUDA_Q3_K: return gran_fmt<KRK_CUDA_Q3_K>(n_in, banks);
    case KRK_CUDA_IQ4_NL: return gran_fmt<KRK_CUDA_IQ4_NL>(n_in, banks);
    case KRK_CUDA_Q5_0: return gran_fmt<KRK_CUDA_Q5_0>(n_in, banks);
    case KRK_CUDA_Q5_1: return gran_fmt<KRK_CUDA_Q5_1>(n_in, banks);
    default: return 0;
    }
}

} // namespace krk_cuda
