"""The prefill GEMM entry that allocates nothing (krk_cuda_gemm_f32_static), against the regular entry.

Collected last on purpose: it is the one test of an add-on entry point, so a run that stops at the first
failure has already been through everything else. It must also pass alone in a fresh process, where its
first call is the very first use of the library on the device.
"""
import numpy as np
import pytest

from kraken_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_scratch_gemm_matches_workspace_gemm_twice(cuda, oracle):
    import torch
    seed = synth.BASE_SEED + 90
    wt = synth.Q4_K
    # Calls in a row, each smaller than the one before: none may see an earlier call's leftovers. The
    # third has an output width that is not a multiple of four and the fourth an output that starts four
    # bytes off a 16-byte boundary: both leave Y by plain stores instead of tensor stores.
    for call, (rows, n_out, n_in, y_shift) in enumerate(((300, 520, 1024, 0), (48, 200, 512, 0), (40, 201, 512, 0),
                                                         (33, 200, 512, 1))):
        w_np = synth.weights(wt, n_out, n_in, seed + call)
        x_np = synth.activations(rows, n_in, seed + call)
        w = torch.from_numpy(w_np).cuda()
        x = torch.from_numpy(x_np).cuda()
        flat = torch.empty(rows * n_out + 4, dtype=torch.float32, device="cuda")
        out = flat[y_shift:y_shift + rows * n_out].view(rows, n_out)
        assert out.data_ptr() % 16 == (4 * y_shift) % 16
        got = cuda.gemm_f32_static(x, w, wt, n_out, n_in, out=out)
        want = cuda.gemm(x, w, wt, n_out, n_in)            # the existing entry, caller-provided workspace
        torch.cuda.synchronize()
        assert cuda.gemm_f32_static_status() == 0
        # and against the CPU checker on the same activations rounded to f16, at the GEMM tests' bound
        x16 = x_np.astype(np.float16).astype(np.float32)
        ref = oracle.gemm(x16, w_np, wt, n_out, n_in, rows=rows, threads=4)
        wd = oracle.dequant_rows(w_np, wt, n_out, n_in).astype(np.float64)
        lim = 2e-3 * np.sqrt((x16.astype(np.float64) ** 2).sum(axis=1))[:, None] * np.sqrt((wd ** 2).sum(axis=1))[None, :]
        assert (np.abs(got.cpu().numpy().astype(np.float64) - ref) <= lim).all()
        # same kernels on the same f16 copy of X: the tolerance of the GEMM tests (2e-3 of ||w_row||*||x_row||)
        # is met with room to spare; in practice the two agree bit for bit
        w_norm = torch.linalg.vector_norm(cuda.dequant_rows(w, wt, n_out, n_in).double(), dim=1)
        x_norm = torch.linalg.vector_norm(x.double(), dim=1)
        bound = 2e-3 * x_norm[:, None] * w_norm[None, :]
        assert bool(((got.double() - want.double()).abs() <= bound).all())
        assert torch.isfinite(got).all()
    # beyond the fixed array: refused with its own code, nothing launched
    before = cuda.launch_count()
    big_rows, big_k = 2048, 4096
    xb = torch.zeros((big_rows, big_k), device="cuda")
    wb = torch.zeros((128, synth.row_bytes(wt, big_k)), dtype=torch.uint8, device="cuda")
    with pytest.raises(cuda.KrkCudaError) as e:
        cuda.gemm_f32_static(xb, wb, wt, 128, big_k)
    assert e.value.rc == -10 and "fixed scratch" in str(e.value)
    assert cuda.launch_count() == before
