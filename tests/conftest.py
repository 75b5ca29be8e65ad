import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """The CPU checker (C restatement of the reference's scalar path)."""
    from oracle.krk_oracle import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The compiled reference, when oracle/_ref was built in this tree."""
    from oracle.krk_oracle import Reference
    if not Reference.available():
        pytest.skip("oracle/_ref/libkrk_ref.so not built here")
    return Reference(threads=2)


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_vectors.npz"))


@pytest.fixture(scope="session")
def cuda():
    """The product library on cuda:0. No fallback: a missing library or device is a failure."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test running without a CUDA device"
    torch.cuda.set_device(0)
    from kraken_b200 import capi
    return capi


def bound_ok(y, y_ref, w_deq, x, tol):
    """|y - y_ref| <= tol * ||w_row||_2 * ||x_row||_2 for every (row, output)."""
    wn = np.sqrt((w_deq.astype(np.float64) ** 2).sum(axis=1))          # [n_out]
    xn = np.sqrt((x.astype(np.float64) ** 2).sum(axis=1))              # [rows]
    lim = tol * xn[:, None] * wn[None, :]
    err = np.abs(y.astype(np.float64) - y_ref.astype(np.float64))
    worst = float((err / np.maximum(lim, 1e-300)).max()) if err.size else 0.0
    return bool((err <= lim).all()), worst
