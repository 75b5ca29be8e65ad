"""The seeded input generator: layouts, distributions, shard-sliceability (no GPU)."""
import numpy as np
import pytest

from kraken_b200 import synth


@pytest.mark.parametrize("wt", synth.FORMATS)
def test_row_slices_equal_full_matrix(wt):
    full = synth.weights(wt, 24, 768, seed=11, stream=3)
    assert full.shape == (24, synth.row_bytes(wt, 768))
    part = synth.weights(wt, 7, 768, seed=11, stream=3, row_begin=9)
    assert np.array_equal(part, full[9:16])
    assert not np.array_equal(synth.weights(wt, 24, 768, seed=12, stream=3), full)
    assert not np.array_equal(synth.weights(wt, 24, 768, seed=11, stream=4), full)


def test_k4_packing_is_inverse_of_reference_unpack(oracle):
    sc = np.arange(8, dtype=np.uint8) * 9 % 64
    mn = (np.arange(8, dtype=np.uint8) * 7 + 5) % 64
    packed = synth.pack_scales_k4(sc[None], mn[None])[0]
    blk = np.zeros(144, np.uint8)
    blk[0:2] = np.array([1.0], np.float16).view(np.uint8)      # d = 1
    blk[2:4] = np.array([1.0], np.float16).view(np.uint8)      # dmin = 1
    blk[4:16] = packed
    blk[16:144] = 0x11                                         # every q = 1 -> value = sc - mn
    v = oracle.dequant_rows(blk, synth.Q4_K, 1, 256)[0].reshape(8, 32)
    assert np.array_equal(v[:, 0], sc.astype(np.float32) - mn.astype(np.float32))


def test_field_distributions(oracle):
    n_in = 4096
    w = synth.weights(synth.Q8_0, 64, n_in, seed=5).reshape(64, -1, 34)
    d = w[..., 0:2].copy().view(np.float16).astype(np.float32)
    q = w[..., 2:].view(np.int8)
    assert d.min() >= 9.9e-4 and d.max() <= 2.0e-2 + 1e-5 and q.min() == -127 and q.max() == 127
    w = synth.weights(synth.Q4_K, 64, n_in, seed=5).reshape(64, -1, 144)
    d = w[..., 0:2].copy().view(np.float16).astype(np.float32)
    dm = w[..., 2:4].copy().view(np.float16).astype(np.float32)
    assert 9.9e-4 <= d.min() and d.max() <= 1.0e-2 + 1e-5 and 0 <= dm.min() and dm.max() <= 5.0e-3 + 1e-5
    w = synth.weights(synth.Q6_K, 64, n_in, seed=5).reshape(64, -1, 210)
    sc = w[..., 192:208].view(np.int8)
    d = w[..., 208:210].copy().view(np.float16).astype(np.float32)
    assert sc.min() == -64 and sc.max() == 63 and 9.9e-5 <= d.min() and d.max() <= 2.0e-3 + 1e-6
    for wt in synth.FORMATS:
        for rp in (False, True):
            deq = oracle.dequant_rows(synth.weights(wt, 8, 1024, seed=5, random_payload=rp), wt, 8, 1024)
            assert np.isfinite(deq).all()


def test_activations():
    x = synth.activations(4, 4096, seed=3)
    assert x.dtype == np.float32 and abs(x.mean()) < 0.05 and abs(x.std() - 1.0) < 0.05
    assert np.array_equal(synth.activations(4, 4096, seed=3), x)
    h = synth.activations_f16(4, 4096, seed=3)
    assert h.dtype == np.float16 and np.array_equal(h, x.astype(np.float16))
