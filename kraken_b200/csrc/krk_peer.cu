// All-gather of partial sums over NVLink peer stores fused with the rank-ordered sum that follows it: the
// exchange step of an expert-sharded FFN (each GPU holds the partial sum of the picks whose experts it
// owns; the result is ((p0 + p1) + p2) + ... in rank order, identical bits on every GPU).
//
// One kernel per step. Phase 1: every CTA copies its share of this GPU's partial sum into slot `my_rank`
// of EVERY GPU's gather buffer (plain 16-byte stores to peer memory; nothing is loaded from a peer), and
// the CTA that finishes last publishes the step's epoch into a flag word on every GPU. Phase 2: every CTA
// waits, bounded, until all peers' epochs have arrived in this GPU's flag words, then adds the slots of its
// own gather buffer in rank order. Steps are counted on the device (the count sits behind the flag words),
// so a launch carries no per-step value and replays from a CUDA graph; the gather buffer is two-deep
// (epoch parity) so that a fast GPU's next step never lands in slots a slow GPU is still adding.
//
// The reference is single-device (src/hip/backend_hip.hip:5036-5043); this has no counterpart there.

#include "krk_common.cuh"

namespace krk_cuda {

namespace {

constexpr long long kPeerWaitCycles = 4000000000LL;   // ~2 s at boost clock, then give up

struct PeerGather {
    float *gather[KRK_CUDA_MAX_PEERS];   // each GPU's buffer: [2][n_peers][slot_stride] floats
    int *flag[KRK_CUDA_MAX_PEERS];       // each GPU's flags: [n_peers] epochs + [1] step count + [1] count of CTAs done
    int n_peers, my_rank;
    long long slot_stride;
};

__global__ void __launch_bounds__(256)
allgather_sum_kernel(PeerGather pg, const float4 *__restrict__ part, float4 *__restrict__ out, long long n4, int *status) {
    int *own = pg.flag[pg.my_rank];
    // CTAs that have stored their share: one word per exchange object, behind its step count, so that two
    // exchanges on one GPU (other streams, other layers) never mix their counts
    unsigned *done_counter = reinterpret_cast<unsigned *>(own + pg.n_peers + 1);
    // every CTA reads the count before it reports below; the last reporter is the only writer
    const int epoch = *reinterpret_cast<volatile int *>(own + pg.n_peers) + 1;
    const size_t half = (size_t)(epoch & 1) * pg.n_peers * pg.slot_stride;
    const size_t mine = half + (size_t)pg.my_rank * pg.slot_stride;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = part[i];
        for (int q = 0; q < pg.n_peers; q++) reinterpret_cast<float4 *>(pg.gather[q] + mine)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(done_counter, 1u);
        if (done == gridDim.x - 1) {
            *done_counter = 0;
            own[pg.n_peers] = epoch;
            __threadfence_system();
            for (int q = 0; q < pg.n_peers; q++) *reinterpret_cast<volatile int *>(pg.flag[q] + pg.my_rank) = epoch;
            __threadfence_system();
        }
    }
    if (threadIdx.x < pg.n_peers) {
        const long long t0 = clock64();
        while (*reinterpret_cast<const volatile int *>(own + threadIdx.x) < epoch) {
            __nanosleep(100);
            if (clock64() - t0 > kPeerWaitCycles) {
                atomicExch(status, KRK_CUDA_ETIMEOUT);
                break;
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    const float4 *slots = reinterpret_cast<const float4 *>(pg.gather[pg.my_rank] + half);
    const long long slot4 = pg.slot_stride / 4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        float4 s = __ldcg(slots + i);
        for (int p = 1; p < pg.n_peers; p++) {
            const float4 v = __ldcg(slots + (long long)p * slot4 + i);
            s.x = __fadd_rn(s.x, v.x);
            s.y = __fadd_rn(s.y, v.y);
            s.z = __fadd_rn(s.z, v.z);
            s.w = __fadd_rn(s.w, v.w);
        }
        out[i] = s;
    }
}

} // namespace

int launch_allgather_sum(float *const gather[], int *const flag[], int n_peers, int my_rank, int64_t slot_stride,
                         const float *part, float *out, int64_t n, cudaStream_t st) {
    if (n == 0) return KRK_CUDA_OK;
    int *status = device_status_word();
    if (!status) return KRK_CUDA_EDEVICE;
    PeerGather pg;
    for (int q = 0; q < n_peers; q++) {
        pg.gather[q] = gather[q];
        pg.flag[q] = flag[q];
    }
    pg.n_peers = n_peers;
    pg.my_rank = my_rank;
    pg.slot_stride = slot_stride;
    const int64_t n4 = n / 4;
    // Every CTA waits for the peers in phase 2 and the publish needs every CTA to have passed phase 1, so
    // the grid never exceeds what is resident at once: one CTA per SM at most.
    const int64_t want = (n4 + 255) / 256;
    const int grid = (int)(want < (int64_t)sm_count() ? want : (int64_t)sm_count());
    allgather_sum_kernel<<<grid, 256, 0, st>>>(pg, reinterpret_cast<const float4 *>(part), reinterpret_cast<float4 *>(out), n4,
                                               status);
    note_launch();
    return check_launch();
}

} // namespace krk_cuda
