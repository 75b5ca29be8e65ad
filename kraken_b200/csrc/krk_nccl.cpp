// NCCL all-gather of the slices of a row-sharded output (or of expert-sharded partial sums) for a C/C++
// host: the reference is single-device, so this replaces nothing there; it is the exchange step of the
// sharded head / expert bank for hosts that do not go through Python. The NCCL library is looked up at run
// time (libnccl.so.2, the copy the process already has when its host linked one), so the CUDA library
// itself carries no link-time dependency on it.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>

#include "krk_cuda.h"

namespace {

struct NcclApi {
    ncclResult_t (*get_unique_id)(ncclUniqueId *) = nullptr;
    ncclResult_t (*comm_init_rank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*comm_destroy)(ncclComm_t) = nullptr;
    ncclResult_t (*all_gather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*error_string)(ncclResult_t) = nullptr;
    bool ok = false;
};

const NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.get_unique_id = reinterpret_cast<decltype(api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
        api.comm_init_rank = reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
        api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
        api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(h, "ncclAllGather"));
        api.error_string = reinterpret_cast<decltype(api.error_string)>(dlsym(h, "ncclGetErrorString"));
        api.ok = api.get_unique_id && api.comm_init_rank && api.comm_destroy && api.all_gather;
    });
    return api;
}

thread_local char g_nccl_err[160] = "";

int fail(ncclResult_t r) {
    const NcclApi &n = nccl();
    const char *text = n.error_string ? n.error_string(r) : "NCCL error";
    std::strncpy(g_nccl_err, text, sizeof(g_nccl_err) - 1);
    g_nccl_err[sizeof(g_nccl_err) - 1] = 0;
    return KRK_CUDA_ELAUNCH;
}

} // namespace

extern "C" {

const char *krk_cuda_nccl_last_error(void) { return g_nccl_err; }

int krk_cuda_nccl_unique_id(unsigned char id[KRK_CUDA_NCCL_ID_BYTES]) {
    static_assert(KRK_CUDA_NCCL_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "id size");
    if (!id) return KRK_CUDA_ENULL;
    const NcclApi &n = nccl();
    if (!n.ok) return KRK_CUDA_EDEVICE;
    ncclUniqueId u;
    const ncclResult_t r = n.get_unique_id(&u);
    if (r != ncclSuccess) return fail(r);
    std::memcpy(id, u.internal, NCCL_UNIQUE_ID_BYTES);
    return KRK_CUDA_OK;
}

int krk_cuda_nccl_comm_init(void **comm, int n_ranks, int rank, const unsigned char id[KRK_CUDA_NCCL_ID_BYTES]) {
    if (!comm || !id) return KRK_CUDA_ENULL;
    if (n_ranks < 1 || rank < 0 || rank >= n_ranks) return KRK_CUDA_EARG;
    const NcclApi &n = nccl();
    if (!n.ok) return KRK_CUDA_EDEVICE;
    ncclUniqueId u;
    std::memcpy(u.internal, id, NCCL_UNIQUE_ID_BYTES);
    ncclComm_t c = nullptr;
    const ncclResult_t r = n.comm_init_rank(&c, n_ranks, u, rank);
    if (r != ncclSuccess) return fail(r);
    *comm = c;
    return KRK_CUDA_OK;
}

int krk_cuda_nccl_comm_destroy(void *comm) {
    if (!comm) return KRK_CUDA_OK;
    const NcclApi &n = nccl();
    if (!n.ok) return KRK_CUDA_EDEVICE;
    const ncclResult_t r = n.comm_destroy(static_cast<ncclComm_t>(comm));
    return r == ncclSuccess ? KRK_CUDA_OK : fail(r);
}

int krk_cuda_shard_allgather(void *full, const void *slice, size_t slice_bytes, void *nccl_comm, void *stream) {
    if (slice_bytes == 0) return KRK_CUDA_OK;
    if (!full || !slice || !nccl_comm) return KRK_CUDA_ENULL;
    const NcclApi &n = nccl();
    if (!n.ok) return KRK_CUDA_EDEVICE;
    // bytes, so that any slice type gathers; in place when slice == full + rank * slice_bytes
    const ncclResult_t r = n.all_gather(slice, full, slice_bytes, ncclInt8, static_cast<ncclComm_t>(nccl_comm),
                                        static_cast<cudaStream_t>(stream));
    return r == ncclSuccess ? KRK_CUDA_OK : fail(r);
}

} // extern "C"
