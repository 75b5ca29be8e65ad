// placeholder until the streaming kernel lands
#include "krk_common.cuh"
namespace krk_cuda {
int launch_gemv_stream(const GemvMat *, int, int64_t, int, int, int, cudaStream_t) { return 0; }
}
