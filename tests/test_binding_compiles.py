"""The Kraken-side binding (include/krk_cuda_kraken_binding.hpp: `class CudaBackend final : public krk::Backend`)
against the reference's own include/krk/backend.hpp: the compiler, not a reader, says that every pure virtual
is overridden with the reference's signature and that the class instantiates, and the program links against
libkrk_cuda.so. Needs the reference tree (KRK_REF, or a directory `reference` beside this repository); skipped
where it is not mounted, e.g. on the GPU box."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PROGRAM = r"""
#include "krk_cuda_kraken_binding.hpp"
#include <cstdio>
#include <type_traits>
// Three helpers of Kraken's own runtime (src/common.cpp) that inline members of the base class call: a
// Kraken build links the real ones; this program only needs the symbols to exist.
namespace krk {
void log_printf(Log, const char *, ...) {}
void *host_alloc(size_t bytes, size_t) { return std::malloc(bytes); }
void host_free(void *p) { std::free(p); }
}
static_assert(!std::is_abstract<krk::CudaBackend>::value, "a pure virtual of krk::Backend is not overridden");
static_assert(std::is_base_of<krk::Backend, krk::CudaBackend>::value, "not a krk::Backend");
int main() {
    std::string err;
    krk::Backend *be = krk::make_cuda_backend(0, &err);   // make_hip_backend's contract: nullptr and a message
    if (!be) { std::printf("no device: %s\n", err.c_str()); return err.empty() ? 12 : 3; }
    const bool ok = be->gemm_k_ok(4096) && !be->gemm_k_ok(100) && be->act_type() == krk::DType::F32 &&
                    be->router_softmax_supported() && be->router_topk_supported() && !be->moe_dispatch_supported();
    std::printf("%s\n", be->describe().c_str());
    delete be;
    return ok ? 0 : 13;
}
"""


def reference_include():
    ref = os.environ.get("KRK_REF") or os.path.join(os.path.dirname(ROOT), "reference")   # a Kraken tree beside this one
    inc = os.path.join(ref, "include")
    return inc if os.path.exists(os.path.join(inc, "krk", "backend.hpp")) else None


def test_binding_compiles_against_the_reference_header_and_links(tmp_path):
    inc = reference_include()
    cxx = shutil.which("g++")
    if inc is None or cxx is None:
        pytest.skip("reference tree (or g++) not present here")
    lib_dir = os.path.join(ROOT, "kraken_b200")
    if not os.path.exists(os.path.join(lib_dir, "libkrk_cuda.so")):
        from kraken_b200 import build
        build.build()
    src = tmp_path / "binding.cpp"
    src.write_text(PROGRAM)
    exe = str(tmp_path / "binding")
    cmd = [cxx, "-std=gnu++17", "-O0", "-Wall", "-Werror=overloaded-virtual", "-I", os.path.join(ROOT, "include"), "-I", inc,
           str(src), "-L", lib_dir, "-lkrk_cuda", f"-Wl,-rpath,{lib_dir}", "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    import torch
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    if torch.cuda.is_available():
        assert run.returncode == 0, (run.returncode, run.stdout, run.stderr)
    else:
        assert run.returncode == 3 and "no device:" in run.stdout, (run.returncode, run.stdout, run.stderr)
