"""The prefill GEMM entry that allocates nothing (krk_cuda_gemm_f32_static), against the regular entry.

Collected last on purpose: it is the one test of an add-on entry point, so a run that stops at the first
failure has already been through everything else. It must also pass alone in a fresh process, where its
first call is the very first use of the library on the device.
"""
import numpy as np
import pytest

from kraken_b200 import synth

pytestmark = pytest.mark.gpu


def test_static_scratch_gemm_matches_workspace_gemm_twice(cuda):
    import torch
    seed = synth.BASE_SEED + 90
    wt = synth.Q4_K
    # two calls in a row, the second smaller than the first: it must not see the first call's leftovers
    for call, (rows, n_out, n_in) in enumerate(((300, 520, 1024), (48, 200, 512))):
        w = torch.from_numpy(synth.weights(wt, n_out, n_in, seed + call)).cuda()
        x = torch.from_numpy(synth.activations(rows, n_in, seed + call)).cuda()
        got = cuda.gemm_f32_static(x, w, wt, n_out, n_in)
        want = cuda.gemm(x, w, wt, n_out, n_in)            # the existing entry, caller-provided workspace
        torch.cuda.synchronize()
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
