"""Seeded synthetic GGUF blocks and activations.

These stand in for real checkpoints (Llama-2-7B / Qwen3-MoE shapes): only the shapes
and the per-field value distributions are reproduced, no real weights.

The generator is counter based: word ``j`` of block ``b`` of row ``r`` of tensor
``stream`` is ``mix64(key(seed, stream) + (global_word_index + 1) * GOLDEN)``. Any row
range of a matrix can therefore be produced on its own (a shard generates exactly its
slice of the full matrix), and the CPU checker and the GPU path consume byte-identical
inputs because both are handed the arrays made here.

Scale fields are written as f16 BIT PATTERNS once, here; neither side re-encodes them
(the reference's ``fp32_to_fp16`` is not exactly round-to-nearest-even on ties,
src/common.cpp:209, so an independent re-encode could differ by one ulp).

Block layouts follow the reference's host decoders: Q8_0 src/quant.cpp:381-387, Q4_0
:331-339, Q4_K :427-460, Q6_K :491-512.
"""
from __future__ import annotations

import numpy as np

Q4_0, Q8_0, Q4_K, Q6_K = 2, 8, 12, 14
Q5_0, Q5_1, Q5_K = 6, 7, 13          # the further formats of mixed files
Q2_K, Q3_K, IQ4_NL = 10, 11, 20
FORMATS = (Q8_0, Q4_0, Q4_K, Q6_K)
MORE_FORMATS = (Q5_0, Q5_1, Q5_K, Q2_K, Q3_K, IQ4_NL)
NAMES = {Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K", Q5_0: "Q5_0", Q5_1: "Q5_1", Q5_K: "Q5_K",
         Q2_K: "Q2_K", Q3_K: "Q3_K", IQ4_NL: "IQ4_NL"}
BLOCK_SIZE = {Q4_0: 32, Q8_0: 32, Q4_K: 256, Q6_K: 256, Q5_0: 32, Q5_1: 32, Q5_K: 256, Q2_K: 256, Q3_K: 256, IQ4_NL: 32}
BLOCK_BYTES = {Q4_0: 18, Q8_0: 34, Q4_K: 144, Q6_K: 210, Q5_0: 22, Q5_1: 24, Q5_K: 176, Q2_K: 84, Q3_K: 110, IQ4_NL: 18}
# 64-bit words of randomness drawn per block
_WORDS = {Q4_0: 3, Q8_0: 9, Q4_K: 19, Q6_K: 27, Q5_0: 4, Q5_1: 4, Q5_K: 23, Q2_K: 11, Q3_K: 15, IQ4_NL: 3}

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_STREAM = np.uint64(0xD1B54A32D192ED03)

BASE_SEED = 0x4B52414B454E0000  # "KRAKEN\0\0"; add the config id


def row_bytes(wt: int, n_in: int) -> int:
    """Bytes of one weight row (src/quant.cpp:1805-1900: rows are unpadded)."""
    bs = BLOCK_SIZE[wt]
    if n_in % bs:
        raise ValueError(f"n_in={n_in} is not a whole number of {NAMES[wt]} blocks")
    return n_in // bs * BLOCK_BYTES[wt]


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def _words(seed: int, stream: int, first: int, count: int) -> np.ndarray:
    """``count`` 64-bit words starting at global word index ``first``."""
    with np.errstate(over="ignore"):
        key = _mix64(np.array([seed & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64)
                     + np.uint64(stream & 0xFFFFFFFFFFFFFFFF) * _STREAM)[0]
        idx = np.arange(first + 1, first + 1 + count, dtype=np.uint64)
        return _mix64(key + idx * _GOLDEN)


def _unit(u32: np.ndarray) -> np.ndarray:
    """uint32 -> float64 in [0, 1)."""
    return u32.astype(np.float64) * (1.0 / 4294967296.0)


def _f16_bits(lo: float, hi: float, u32: np.ndarray) -> np.ndarray:
    """Uniform value in [lo, hi] rounded once to f16 (numpy: IEEE nearest-even)."""
    v = lo + (hi - lo) * _unit(u32)
    return v.astype(np.float16).view(np.uint16)


def _put_u16(blocks: np.ndarray, off: int, bits: np.ndarray) -> None:
    blocks[..., off] = (bits & 0xFF).astype(np.uint8)
    blocks[..., off + 1] = (bits >> 8).astype(np.uint8)


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of the reference's 6-bit unpack (src/quant.cpp:427-435).

    sc, mn: uint8 arrays [..., 8] with values 0..63 -> uint8 [..., 12].
    """
    out = np.zeros(sc.shape[:-1] + (12,), dtype=np.uint8)
    out[..., 0:4] = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 0xF) | ((mn[..., 4:8] & 0xF) << 4)
    return out


def weights(wt: int, n_rows: int, n_in: int, seed: int, stream: int = 0, row_begin: int = 0,
            random_payload: bool = False) -> np.ndarray:
    """Rows ``[row_begin, row_begin + n_rows)`` of a synthetic quantized matrix.

    Returns uint8 ``[n_rows, row_bytes]``. With ``random_payload`` every non-scale byte
    is uniform 0..255 (every byte pattern is a legal block, which is how the
    reference's own probes build K-quant fixtures: tools/bench_ops.cpp:92-141); the
    f16 scale slots keep benign values either way.
    """
    nblk = n_in // BLOCK_SIZE[wt]
    row_bytes(wt, n_in)
    nw = _WORDS[wt]
    w = _words(seed, stream, row_begin * nblk * nw, n_rows * nblk * nw).reshape(n_rows, nblk, nw)
    by = w.view(np.uint8).reshape(n_rows, nblk, nw * 8)  # little-endian bytes of the words
    blocks = np.zeros((n_rows, nblk, BLOCK_BYTES[wt]), dtype=np.uint8)
    hdr = w[..., nw - 1]
    u_lo = (hdr & np.uint64(0xFFFFFFFF)).astype(np.uint32)
    u_hi = (hdr >> np.uint64(32)).astype(np.uint32)
    if wt == Q8_0:
        _put_u16(blocks, 0, _f16_bits(1e-3, 2e-2, u_lo))
        if random_payload:
            blocks[..., 2:34] = by[..., 0:32]
        else:
            h = np.ascontiguousarray(w[..., 0:8]).view(np.uint16).reshape(n_rows, nblk, 32).astype(np.uint32)
            blocks[..., 2:34] = (((h * 255) >> 16).astype(np.int32) - 127).astype(np.int8).view(np.uint8)
    elif wt == Q4_0:
        _put_u16(blocks, 0, _f16_bits(1e-3, 2e-2, u_lo))
        blocks[..., 2:18] = by[..., 0:16]
    elif wt == Q4_K:
        _put_u16(blocks, 0, _f16_bits(1e-3, 1e-2, u_lo))
        _put_u16(blocks, 2, _f16_bits(0.0, 5e-3, u_hi))
        if random_payload:
            blocks[..., 4:16] = by[..., 128:140]
        else:
            six = by[..., 128:144] & 63
            blocks[..., 4:16] = pack_scales_k4(six[..., 0:8], six[..., 8:16])
        blocks[..., 16:144] = by[..., 0:128]
    elif wt == Q6_K:
        blocks[..., 0:192] = by[..., 0:192]  # ql and qh: uniform bits <=> 6-bit q uniform in 0..63
        if random_payload:
            blocks[..., 192:208] = by[..., 192:208]
        else:
            blocks[..., 192:208] = ((by[..., 192:208] & 127).astype(np.int16) - 64).astype(np.int8).view(np.uint8)
        _put_u16(blocks, 208, _f16_bits(1e-4, 2e-3, u_lo))
    elif wt == Q5_0:      # d, 4 bytes of fifth bits, 16 bytes of nibbles: every payload byte uniform
        _put_u16(blocks, 0, _f16_bits(1e-3, 2e-2, u_lo))
        blocks[..., 2:22] = by[..., 0:20]
    elif wt == Q5_1:      # d, offset m, fifth bits, nibbles
        _put_u16(blocks, 0, _f16_bits(1e-3, 2e-2, u_lo))
        _put_u16(blocks, 2, _f16_bits(-0.2, 0.2, u_hi))
        blocks[..., 4:24] = by[..., 0:20]
    elif wt == Q5_K:      # d, dmin, 12 packed scale bytes, 32 bytes of fifth bits, 128 bytes of nibbles
        _put_u16(blocks, 0, _f16_bits(1e-3, 1e-2, u_lo))
        _put_u16(blocks, 2, _f16_bits(0.0, 5e-3, u_hi))
        if random_payload:
            blocks[..., 4:16] = by[..., 160:172]
        else:
            six = by[..., 160:176] & 63
            blocks[..., 4:16] = pack_scales_k4(six[..., 0:8], six[..., 8:16])
        blocks[..., 16:176] = by[..., 0:160]
    elif wt == Q2_K:      # 16 scale/min bytes, 64 bytes of 2-bit quants, d, dmin: every payload byte uniform
        blocks[..., 0:80] = by[..., 0:80]
        _put_u16(blocks, 80, _f16_bits(1e-3, 1e-2, u_lo))
        _put_u16(blocks, 82, _f16_bits(0.0, 5e-3, u_hi))
    elif wt == Q3_K:      # 32 mask bytes, 64 bytes of 2-bit quants, 12 packed 6-bit scale bytes, d
        blocks[..., 0:108] = by[..., 0:108]
        _put_u16(blocks, 108, _f16_bits(1e-3, 1e-2, u_lo))
    elif wt == IQ4_NL:    # d and 16 bytes of grid indices
        _put_u16(blocks, 0, _f16_bits(1e-4, 2e-3, u_lo))
        blocks[..., 2:18] = by[..., 0:16]
    else:
        raise ValueError(f"unsupported weight type {wt}")
    return blocks.reshape(n_rows, nblk * BLOCK_BYTES[wt])


def normal(n: int, seed: int, stream: int, first: int = 0) -> np.ndarray:
    """``n`` f32 samples of N(0,1): Box-Muller in f64, rounded once to f32."""
    w = _words(seed, stream, first, n)
    u1 = ((w >> np.uint64(32)).astype(np.float64) + 1.0) * (1.0 / 4294967296.0)  # (0, 1]
    u2 = (w & np.uint64(0xFFFFFFFF)).astype(np.float64) * (1.0 / 4294967296.0)
    return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def activations(rows: int, n_in: int, seed: int, stream: int = 1000) -> np.ndarray:
    """f32 ``[rows, n_in]`` ~ N(0,1)."""
    return normal(rows * n_in, seed, stream).reshape(rows, n_in)


def activations_f16(rows: int, n_in: int, seed: int, stream: int = 1000) -> np.ndarray:
    """f16 ``[rows, n_in]``: the f32 samples rounded once (the checker widens these)."""
    return activations(rows, n_in, seed, stream).astype(np.float16)
