"""Prefill GEMM (tcgen05) against the CPU checker, through the C ABI.

Bar: f16-staged operands, so |y - y_ref| <= 2e-3 * ||w_row|| * ||x_row|| with y_ref the scalar f32
reference on the same f16 activations widened to f32.
"""
import numpy as np
import pytest

from conftest import bound_ok
from kraken_b200 import synth

pytestmark = pytest.mark.gpu

GEMM_TOL = 2e-3
SEED = synth.BASE_SEED + 3


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_gemm(cuda, oracle, wt, n_out, n_in, rows, seed, f32_x=False, check_rows=None):
    before = cuda.family_count(cuda.FAMILY_GEMM_TC)
    w = synth.weights(wt, n_out, n_in, seed, stream=wt)
    x16 = synth.activations_f16(rows, n_in, seed)
    x = x16.astype(np.float32)
    y = cuda.gemm(dev(x if f32_x else x16), dev(w), wt, n_out, n_in).cpu().numpy()
    assert cuda.device_status() == 0
    assert cuda.family_count(cuda.FAMILY_GEMM_TC) == before + 1
    sel = np.arange(n_out) if check_rows is None else check_rows
    y_ref = oracle.gemm(x, w[sel], wt, len(sel), n_in, rows=rows, threads=8)
    w_deq = oracle.dequant_rows(w[sel], wt, len(sel), n_in)
    ok, worst = bound_ok(y[:, sel], y_ref, w_deq, x, GEMM_TOL)
    assert ok, f"wt={wt} {rows}x{n_out}x{n_in}: worst error is {worst:.3f} of the bound"
    return worst


def test_gemm_smallest_first(cuda, oracle):
    """One tile, one K block: the first thing to run on a fresh build."""
    run_gemm(cuda, oracle, synth.Q4_K, 128, 256, 16, SEED)
    run_gemm(cuda, oracle, synth.Q4_K, 128, 1024, 64, SEED + 1)


@pytest.mark.parametrize("wt", [synth.Q4_K, synth.Q8_0, synth.Q6_K, synth.Q4_0, synth.Q5_K, synth.Q5_0])
def test_gemm_tile_boundaries(cuda, oracle, wt):
    # the reference suite's row counts around its tile edges (tests/test_kraken.cpp:759), plus ours
    for rows in (9, 13, 16, 37, 255, 256, 257):
        run_gemm(cuda, oracle, wt, 200, 512, rows, SEED + rows)
    run_gemm(cuda, oracle, wt, 129, 256, 300, SEED + 50)
    run_gemm(cuda, oracle, wt, 1000, 1024, 130, SEED + 51)
    # an odd number of 256-value blocks per row (Q6_K rows then start on every other 2-byte boundary), and
    # enough K for the staging ring to wrap several times
    run_gemm(cuda, oracle, wt, 131, 768, 20, SEED + 52)
    run_gemm(cuda, oracle, wt, 260, 4352, 33, SEED + 53)


def test_gemm_f32_activations(cuda, oracle):
    run_gemm(cuda, oracle, synth.Q4_K, 384, 1024, 40, SEED + 60, f32_x=True)


def test_gemm_many_tiles_per_cta(cuda, oracle):
    # more tiles than SMs, so every CTA walks several tiles and both accumulator buffers wrap
    run_gemm(cuda, oracle, synth.Q4_K, 128 * 200, 256, 520, SEED + 61, check_rows=np.arange(0, 128 * 200, 97))


@pytest.mark.parametrize("rows", [128, 512, 2048])
def test_config3_q4_k_prefill(cuda, oracle, rows):
    """N = 14336, K = 4096, M in {128, 512, 2048}; the checker runs on every 29th weight row."""
    run_gemm(cuda, oracle, synth.Q4_K, 14336, 4096, rows, SEED + 70, check_rows=np.arange(0, 14336, 29))


def test_gemm_refusals(cuda):
    import torch
    x = torch.zeros((16, 256), dtype=torch.float16, device="cuda")
    w = torch.zeros(144 * 128, dtype=torch.uint8, device="cuda")
    with pytest.raises(cuda.KrkCudaError) as e:
        cuda.gemm(x[:, :96].contiguous(), w, synth.Q8_0, 128, 96)     # K must be a multiple of 256
    assert e.value.rc == -2
    y = torch.empty((16, 128), device="cuda")
    rc = cuda.lib.krk_cuda_gemm(y.data_ptr(), x.float().data_ptr(), cuda.X_F32, w.data_ptr(), synth.Q4_K, 128, 256, 16,
                                None, 0, None)
    assert rc == -6                                                   # f32 X needs a workspace
    assert cuda.gemm(x[:0], w, synth.Q4_K, 128, 256).shape == (0, 128)


def test_backend_gemm_rows_over_8_uses_tensor_cores(cuda, oracle):
    be = cuda.Backend(0)
    n_out, n_in, rows = 300, 512, 24
    w = synth.weights(synth.Q4_K, n_out, n_in, SEED + 80)
    x = synth.activations_f16(rows, n_in, SEED + 80).astype(np.float32)
    d_w, d_x, d_y = be.alloc(w.nbytes), be.alloc(x.nbytes), be.alloc(rows * n_out * 4)
    be.upload(d_w, w.ctypes.data, w.nbytes)
    be.upload(d_x, x.ctypes.data, x.nbytes)
    before = cuda.family_count(cuda.FAMILY_GEMM_TC)
    be.gemm(d_y, d_x, d_w, synth.Q4_K, n_out, n_in, rows)
    y = np.empty((rows, n_out), np.float32)
    be.download(y.ctypes.data, d_y, y.nbytes)
    assert cuda.family_count(cuda.FAMILY_GEMM_TC) == before + 1
    ref = oracle.gemm(x, w, synth.Q4_K, n_out, n_in, rows=rows, threads=8)
    ok, worst = bound_ok(y, ref, oracle.dequant_rows(w, synth.Q4_K, n_out, n_in), x, GEMM_TOL)
    assert ok, worst
    for ptr in (d_w, d_x, d_y):
        be.release(ptr)
    be.close()


def test_gemm_cut_tail_tiles_opt_in(oracle):
    """KRK_CUDA_GEMM_SPLIT=1 (read once per process, so a child process): the tiles left after the last
    whole wave are cut over all CTAs and their pieces added in K order; same bar, and bit-identical runs."""
    import os
    import subprocess
    import sys
    import tempfile
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    n_out, n_in, rows = 128 * 150, 512, 300        # 300 tiles on 148 SMs: two whole waves and a cut tail
    code = f"""
import sys, numpy as np, torch
sys.path.insert(0, {root!r})
from kraken_b200 import capi, synth
w = torch.from_numpy(synth.weights(synth.Q4_K, {n_out}, {n_in}, {SEED + 95})).cuda()
x = torch.from_numpy(synth.activations_f16({rows}, {n_in}, {SEED + 95})).cuda()
y1 = capi.gemm(x, w, synth.Q4_K, {n_out}, {n_in})
y2 = capi.gemm(x, w, synth.Q4_K, {n_out}, {n_in})
assert capi.device_status() == 0 and torch.equal(y1, y2)
np.save(sys.argv[1], y1.cpu().numpy())
"""
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "y.npy")
        env = dict(os.environ, KRK_CUDA_GEMM_SPLIT="1")
        subprocess.run([sys.executable, "-c", code, out], check=True, env=env, timeout=300)
        y = np.load(out)
    w = synth.weights(synth.Q4_K, n_out, n_in, SEED + 95)
    x = synth.activations_f16(rows, n_in, SEED + 95).astype(np.float32)
    sel = np.arange(0, n_out, 53)
    ref = oracle.gemm(x, w[sel], synth.Q4_K, len(sel), n_in, rows=rows, threads=8)
    ok, worst = bound_ok(y[:, sel], ref, oracle.dequant_rows(w[sel], synth.Q4_K, len(sel), n_in), x, GEMM_TOL)
    assert ok, worst
