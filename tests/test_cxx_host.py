"""The C++ host side on its own: a program that includes include/krk_cuda_backend.hpp, links the C-ABI library
and drives CudaBackend the way a Kraken build would. Without a GPU make() must return nullptr and fill
`err` (the make_hip_backend contract, include/krk/backend.hpp:1886); with one the numbers must be right."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cxx", "backend_smoke.cpp")


def build_program(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    lib_dir = os.path.join(ROOT, "kraken_b200")
    if not os.path.exists(os.path.join(lib_dir, "libkrk_cuda.so")):
        from kraken_b200 import build
        build.build()
    exe = str(tmp_path / "backend_smoke")
    cmd = [cxx, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), SRC, "-L", lib_dir, "-lkrk_cuda",
           f"-Wl,-rpath,{lib_dir}", "-o", exe]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


def test_cxx_host_without_a_device_gets_nullptr_and_a_message(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present: the device run is the gpu-marked test")
    exe = build_program(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert r.returncode == 3, (r.returncode, r.stdout, r.stderr)
    assert "no device:" in r.stdout and len(r.stdout.strip()) > len("no device:")


@pytest.mark.gpu
def test_cxx_host_runs_a_gemm(tmp_path):
    exe = build_program(tmp_path)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.returncode, r.stdout, r.stderr)
    assert "0 of 40 rows off" in r.stdout
