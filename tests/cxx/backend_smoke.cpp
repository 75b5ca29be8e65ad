// A C++ host driving the backend class directly, the way a Kraken build would (no Python, no torch):
// make() with make_hip_backend's contract, alloc / upload / gemm / download, the C ABI for a refusal.
// Exit codes: 0 = ran on a device and the numbers are right; 3 = no usable device (make() returned nullptr
// and filled `err`, as the contract asks); anything else = a failure.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "krk_cuda.h"
#include "krk_cuda_backend.hpp"

using krk_cuda::CudaBackend;
using krk_cuda::DType;

static uint16_t half_bits(float v) {   // exact for the few constants used here (1.0, 0.5, 0.25)
    uint32_t u;
    std::memcpy(&u, &v, 4);
    return (uint16_t)(((u >> 16) & 0x8000u) | ((((u >> 23) & 0xFFu) - 112u) << 10) | ((u >> 13) & 0x3FFu));
}

int main() {
    // refusals come back as codes before any device is touched
    if (krk_cuda_gemm_k_ok(KRK_CUDA_Q4_K, 100) != 0 || krk_cuda_gemm_k_ok(KRK_CUDA_Q8_0, 4096) != 1) return 10;
    if (std::string(krk_cuda_strerror(KRK_CUDA_ESHAPE)).empty()) return 11;

    std::string err;
    CudaBackend *be = CudaBackend::make(0, &err);
    if (!be) {
        std::printf("no device: %s\n", err.c_str());
        return err.empty() ? 12 : 3;
    }
    // Q8_0, the reference's layout test block (tests/test_kraken.cpp:563-573): d = 0.5, q = i - 16
    const int n_out = 40, n_in = 64, blocks = n_in / 32;
    std::vector<uint8_t> w((size_t)n_out * blocks * 34);
    for (int r = 0; r < n_out; r++)
        for (int b = 0; b < blocks; b++) {
            uint8_t *p = &w[((size_t)r * blocks + b) * 34];
            const uint16_t d = half_bits(r % 2 ? 0.5f : 0.25f);
            p[0] = (uint8_t)(d & 0xFF);
            p[1] = (uint8_t)(d >> 8);
            for (int i = 0; i < 32; i++) p[2 + i] = (uint8_t)(int8_t)(i - 16);
        }
    std::vector<float> x(n_in), y(n_out, -1.0f);
    for (int i = 0; i < n_in; i++) x[i] = (float)((i % 7) - 3);
    void *d_w = be->alloc(w.size()), *d_x = be->alloc(x.size() * 4), *d_y = be->alloc(y.size() * 4);
    be->upload(d_w, w.data(), w.size());
    be->upload(d_x, x.data(), x.size() * 4);
    be->gemm(d_y, d_x, d_w, DType::Q8_0, n_out, n_in, 1);
    be->download(y.data(), d_y, y.size() * 4);
    int bad = 0;
    for (int r = 0; r < n_out; r++) {
        const float d = r % 2 ? 0.5f : 0.25f;
        float want = 0.0f;
        for (int i = 0; i < n_in; i++) want += d * (float)((i % 32) - 16) * x[i];
        if (std::fabs(y[r] - want) > 1e-4f * (std::fabs(want) + 1.0f)) bad++;
    }
    std::printf("%s: %d of %d rows off\n", be->describe(), bad, n_out);
    // the MoE batching helpers: gather two rows of a 3 x 8 matrix, activate them as two one-row buffers
    {
        std::vector<float> m(24), g(16, -7.0f), act(16, -7.0f);
        for (int i = 0; i < 24; i++) m[i] = 0.25f * (float)(i - 9);
        const int32_t pick[2] = {2, 0};
        void *d_m = be->alloc(96), *d_g = be->alloc(64), *d_a = be->alloc(64);
        int32_t *d_pick = static_cast<int32_t *>(be->alloc(8));
        be->upload(d_m, m.data(), 96);
        be->upload_i32(d_pick, pick, 2);
        be->gather_rows(d_g, d_m, d_pick, 2, 8);
        be->download(g.data(), d_g, 64);
        for (int i = 0; i < 8; i++)
            if (g[i] != m[16 + i] || g[8 + i] != m[i]) bad++;
        void *outs[2] = {d_a, static_cast<float *>(d_a) + 8};
        const void *gates[2] = {d_g, static_cast<const float *>(d_g) + 8}, *ups[2] = {d_g, static_cast<const float *>(d_g) + 8};
        float s0 = 0.0f, s1 = 0.0f;
        float *scales[2] = {&s0, &s1};
        be->silu_mul_rows(outs, gates, ups, 8, 2, scales);
        be->download(act.data(), d_a, 64);
        for (int i = 0; i < 16; i++) {
            const float want = g[i] / (1.0f + std::exp(-g[i])) * g[i];
            if (std::fabs(act[i] - want) > 1e-5f * (std::fabs(want) + 1.0f)) bad++;
        }
        if (s0 != 1.0f || s1 != 1.0f) bad++;
        be->release(d_m);
        be->release(d_g);
        be->release(d_a);
        be->release(d_pick);
    }
    be->release(d_w);
    be->release(d_x);
    be->release(d_y);
    delete be;
    return bad ? 20 : 0;
}
