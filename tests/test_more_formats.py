"""The further GGUF formats a mixed file carries (Q5_0, Q5_1, Q5_K, Q2_K, Q3_K, IQ4_NL): bit-exact row decode, the shape-agnostic
GEMV within the decode bar, the prefill GEMM within its bar, embedding gather. The restatement is pinned
against the compiled reference wherever that library is present (it cannot travel to a GPU box)."""
import numpy as np
import pytest

from kraken_b200 import synth
from tests.conftest import bound_ok

FMTS = list(synth.MORE_FORMATS)
SEED = synth.BASE_SEED + 55


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("wt", FMTS)
def test_geometry_and_oracle_known_answers(oracle, wt):
    assert oracle.block_size(wt) == synth.BLOCK_SIZE[wt] and oracle.block_bytes(wt) == synth.BLOCK_BYTES[wt]
    # one hand-built block per format: scale 1.0, all fifth bits set, nibbles 0x0F -> q = 31 (low half), 16 (high half)
    one = np.float16(1.0).view(np.uint16)
    if wt == synth.Q5_0:
        b = np.zeros(22, np.uint8); b[0], b[1] = one & 0xFF, one >> 8; b[2:6] = 0xFF; b[6:22] = 0x0F
        y = oracle.dequant_rows(b, wt, 1, 32)[0]
        assert np.all(y[:16] == 15.0) and np.all(y[16:] == 0.0)          # (31 - 16), (16 - 16)
    elif wt == synth.Q5_1:
        b = np.zeros(24, np.uint8); b[0], b[1] = one & 0xFF, one >> 8
        half = np.float16(0.5).view(np.uint16); b[2], b[3] = half & 0xFF, half >> 8; b[4:8] = 0xFF; b[8:24] = 0x0F
        y = oracle.dequant_rows(b, wt, 1, 32)[0]
        assert np.all(y[:16] == 31.5) and np.all(y[16:] == 16.5)
    elif wt == synth.Q2_K:
        # scale byte 0x23 (scale 3, min 2), every quant 0b11_10_01_00, d = 1, dmin = 0.5: bit pair j gives q = j
        b = np.zeros(84, np.uint8); b[0:16] = 0x23; b[16:80] = 0xE4; b[80], b[81] = one & 0xFF, one >> 8
        half = np.float16(0.5).view(np.uint16); b[82], b[83] = half & 0xFF, half >> 8
        y = oracle.dequant_rows(b, wt, 1, 256)[0]
        for j in range(4):
            assert np.all(y[32 * j:32 * j + 32] == 3.0 * j - 1.0) and np.all(y[128 + 32 * j:160 + 32 * j] == 3.0 * j - 1.0)
    elif wt == synth.Q3_K:
        # all mask bits set (no -4), quants 0b11_10_01_00, scale nibbles 1 with high bits 2: scale = (1 | 2 << 4) - 32 = 1
        b = np.zeros(110, np.uint8); b[0:32] = 0xFF; b[32:96] = 0xE4; b[96:104] = 0x11; b[104:108] = 0xAA
        b[108], b[109] = one & 0xFF, one >> 8
        y = oracle.dequant_rows(b, wt, 1, 256)[0]
        for j in range(4):
            assert np.all(y[32 * j:32 * j + 32] == float(j))
        b[0:32] = 0x00                                                     # every mask bit clear: q - 4
        assert np.all(oracle.dequant_rows(b, wt, 1, 256)[0][:32] == -4.0)
    elif wt == synth.IQ4_NL:
        b = np.zeros(18, np.uint8); b[0], b[1] = one & 0xFF, one >> 8; b[2:18] = 0xF0      # low nibble 0, high nibble 15
        y = oracle.dequant_rows(b, wt, 1, 32)[0]
        assert np.all(y[:16] == -127.0) and np.all(y[16:] == 113.0)      # the ends of the format's grid
    else:
        b = np.zeros(176, np.uint8); b[0], b[1] = one & 0xFF, one >> 8; b[4:16] = 1; b[16:48] = 0x01; b[48:176] = 0x21
        y = oracle.dequant_rows(b, wt, 1, 256)[0]
        # chunk 0: low nibble 1 + fifth bit (mask bit 0) = 17, scale 1; chunk 1: high nibble 2, no fifth bit
        assert np.all(y[:32] == 17.0 - 0.0) and np.all(y[32:64] == 2.0)


@pytest.mark.parametrize("wt", FMTS)
def test_oracle_matches_reference_vectors(oracle, golden, wt):
    name = synth.NAMES[wt].lower()
    w, x = golden[f"{name}_bytes_w"], golden[f"{name}_bytes_x"]
    assert oracle.dequant_rows(w, wt, 5, 1024).tobytes() == golden[f"{name}_bytes_deq"].tobytes()
    assert oracle.gemm(x, w, wt, 5, 1024, rows=2).tobytes() == golden[f"{name}_bytes_y"].tobytes()


@pytest.mark.parametrize("wt", FMTS)
def test_oracle_equals_compiled_reference(oracle, reference, wt):
    for rp in (False, True):
        w = synth.weights(wt, 17, 1024, SEED, stream=wt, random_payload=rp)
        x = synth.activations(2, 1024, SEED)
        assert oracle.dequant_rows(w, wt, 17, 1024).tobytes() == reference.dequant_rows(w, wt, 17, 1024).tobytes()
        assert oracle.gemm(x, w, wt, 17, 1024, rows=2).tobytes() == reference.gemm(x, w, wt, 17, 1024, rows=2, tier=0).tobytes()


@pytest.mark.gpu
@pytest.mark.parametrize("wt", FMTS)
def test_device_decode_gemv_gemm_embed(cuda, oracle, wt):
    import torch
    n_out, n_in = 515, 2048
    for rp in (False, True):
        w = synth.weights(wt, n_out, n_in, SEED + 1, stream=wt, random_payload=rp)
        got = cuda.dequant_rows(dev(w), wt, n_out, n_in).cpu().numpy()
        want = oracle.dequant_rows(w, wt, n_out, n_in)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(np.nan_to_num(got).view(np.uint32), np.nan_to_num(want).view(np.uint32))
    w = synth.weights(wt, n_out, n_in, SEED + 2, stream=wt)
    w_deq = oracle.dequant_rows(w, wt, n_out, n_in)
    for rows in (1, 3, 8):
        x = synth.activations(rows, n_in, SEED + rows)
        y = cuda.gemv(dev(x), dev(w), wt, n_out, n_in).cpu().numpy()
        ok, worst = bound_ok(y, oracle.gemm(x, w, wt, n_out, n_in, rows=rows, threads=8), w_deq, x, 1e-4)
        assert ok, worst
    rows = 40                                                      # the tensor-core path
    x16 = synth.activations(rows, n_in, SEED + 40).astype(np.float16)
    xf = x16.astype(np.float32)
    y = cuda.gemm(dev(x16), dev(w), wt, n_out, n_in).cpu().numpy()
    ok, worst = bound_ok(y, oracle.gemm(xf, w, wt, n_out, n_in, rows=rows, threads=8), w_deq, xf, 2e-3)
    assert ok, worst
    toks = np.array([0, 514, 515, -2, 77], np.int32)
    e = cuda.embed(dev(w), wt, n_out, n_in, dev(toks)).cpu().numpy()
    assert e.tobytes() == oracle.embed(w, wt, n_out, n_in, toks).tobytes()
    assert cuda.device_status() == 0
