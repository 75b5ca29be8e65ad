"""Regenerates tests/golden/*.npz from the reference's own compiled CPU code.

Run in a container where the reference tree is mounted (it cannot travel):

    make -C oracle ref && python tests/golden/make_golden.py

Every array stored here was produced by oracle/_ref/libkrk_ref.so, i.e. by the reference's
unmodified sources (krk::dequant_row, CpuBackend::gemm with the three lossy/reordered tiers
switched off, CpuBackend::silu_mul / scatter_axpy_rows / embed / logits_topk); the inputs are the seeded synthetic
blocks of kraken_b200.synth plus the hand-built blocks of the reference's known-answer tests
(tests/test_kraken.cpp:456-469, 563-573, 981-1001, 1026-1042). Nothing under the reference tree is
read by the tests themselves: they read only the .npz files.
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from kraken_b200 import synth  # noqa: E402
from oracle.krk_oracle import Reference  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
SEED = synth.BASE_SEED + 99

# (n_rows, n_in) per format: odd row counts and a K that is not a power of two
SHAPES = {synth.Q8_0: (7, 1312), synth.Q4_0: (5, 992), synth.Q4_K: (6, 1280), synth.Q6_K: (5, 1536)}


def kat_blocks(ref: Reference):
    """The hand-built blocks of the reference's own layout tests."""
    def f16(v):
        return ref.fp32_to_fp16(v)

    out = {}
    b = np.zeros(18, np.uint8)                       # test_q4_0_layout
    b[0], b[1] = f16(1.0) & 0xFF, f16(1.0) >> 8
    b[2:18] = [(i | (i << 4)) for i in range(16)]
    out["kat_q4_0"] = (synth.Q4_0, b, 32)
    b = np.zeros(34, np.uint8)                       # test_q8_0_layout
    b[0], b[1] = f16(0.5) & 0xFF, f16(0.5) >> 8
    b[2:34] = np.array([i - 16 for i in range(32)], np.int8).view(np.uint8)
    out["kat_q8_0"] = (synth.Q8_0, b, 32)
    b = np.zeros(144, np.uint8)                      # test_kquant_roundtrip_shape
    b[0], b[1] = f16(0.5) & 0xFF, f16(0.5) >> 8
    b[2], b[3] = f16(0.25) & 0xFF, f16(0.25) >> 8
    b[4:16] = 1
    b[16:144] = 0x88
    out["kat_q4_k"] = (synth.Q4_K, b, 256)
    b = np.zeros(210, np.uint8)                      # test_q6_k_group_stride
    b[208], b[209] = f16(1.0) & 0xFF, f16(1.0) >> 8
    b[192:208] = 1
    b[128 + 32] = 0x03
    out["kat_q6_k"] = (synth.Q6_K, b, 256)
    return out


def main():
    ref = Reference(threads=2)
    data = {}
    for wt, (n_rows, n_in) in SHAPES.items():
        name = synth.NAMES[wt].lower()
        for tag, rp in (("field", False), ("bytes", True)):
            w = synth.weights(wt, n_rows, n_in, SEED, stream=wt, random_payload=rp)
            x = synth.activations(3, n_in, SEED, stream=500 + wt)
            data[f"{name}_{tag}_w"] = w
            data[f"{name}_{tag}_x"] = x
            data[f"{name}_{tag}_deq"] = ref.dequant_rows(w, wt, n_rows, n_in)
            data[f"{name}_{tag}_y"] = ref.gemm(x, w, wt, n_rows, n_in, rows=3, tier=0)
    # the further formats of mixed files (decode and exact GEMM of random-payload blocks)
    for wt in synth.MORE_FORMATS:
        name = synth.NAMES[wt].lower()
        w = synth.weights(wt, 5, 1024, SEED, stream=wt, random_payload=True)
        x = synth.activations(2, 1024, SEED, stream=600 + wt)
        data[f"{name}_bytes_w"], data[f"{name}_bytes_x"] = w, x
        data[f"{name}_bytes_deq"] = ref.dequant_rows(w, wt, 5, 1024)
        data[f"{name}_bytes_y"] = ref.gemm(x, w, wt, 5, 1024, rows=2, tier=0)
    for key, (wt, blk, n) in kat_blocks(ref).items():
        data[f"{key}_w"] = blk
        data[f"{key}_deq"] = ref.dequant_rows(blk, wt, 1, n)
    # half -> float over every bit pattern
    data["fp16_table"] = np.array([ref.fp16_to_fp32(h) for h in range(65536)], np.float32).view(np.uint32)
    # MoE-adjacent ops
    g = synth.normal(777, SEED, 900) * 3.0
    u = synth.normal(777, SEED, 901)
    data["silu_gate"], data["silu_up"], data["silu_out"] = g, u, ref.silu_mul(g, u)
    dst = synth.normal(6 * 40, SEED, 902).reshape(6, 40).copy()
    src = synth.normal(3 * 40, SEED, 903).reshape(3, 40)
    rows = np.array([4, 0, 5], np.int32)
    alpha = np.array([0.25, 1.0, -1.5], np.float32)
    data["scatter_dst"], data["scatter_src"], data["scatter_rows"], data["scatter_alpha"] = dst.copy(), src, rows, alpha
    data["scatter_out"] = ref.scatter_axpy_rows(dst, src, rows, alpha)
    # the steps either side of the head: embedding gather (bad ids give zero rows) and top-k of a logits row
    for wt in SHAPES:
        name = synth.NAMES[wt].lower()
        table = synth.weights(wt, 40, 512, SEED, stream=900 + wt)
        toks = np.array([3, 39, -1, 40, 0, 17, 3], np.int32)
        data[f"embed_{name}_table"], data[f"embed_{name}_tokens"] = table, toks
        data[f"embed_{name}_out"] = ref.embed(table, wt, 40, 512, toks)
    lg = synth.normal(5000, SEED, 904) * 4.0
    lg[100] = lg[4000] = lg.max() + 1.0           # an exact tie at the top: the lower id first
    pm = np.zeros((5000 + 31) // 32, np.uint32)
    pm[3], pm[125] = 0xFFFF00FF, 0x00000101        # ids 96..103, 112..127, 4000, 4008 are penalised
    data["topk_logits"], data["topk_mask"] = lg, pm
    for tag, (k, cap, pen, temp) in {"a": (1, 0.0, 1.0, 1.0), "b": (8, 3.0, 1.3, 0.7), "c": (64, 0.0, 1.1, 1.0)}.items():
        ids, vals, mass = ref.logits_topk(lg, k, pm, pen, cap, temp)
        data[f"topk_{tag}_args"] = np.array([k, cap, pen, temp], np.float32)
        data[f"topk_{tag}_ids"], data[f"topk_{tag}_vals"], data[f"topk_{tag}_mass"] = ids, vals, np.float32(mass)
    ids, vals, _ = ref.logits_topk(lg[:5], 8)      # fewer elements than k: -1 / -FLT_MAX markers
    data["topk_short_ids"], data["topk_short_vals"] = ids, vals
    np.savez_compressed(os.path.join(OUT, "reference_vectors.npz"), **data)
    print("wrote", os.path.join(OUT, "reference_vectors.npz"),
          os.path.getsize(os.path.join(OUT, "reference_vectors.npz")), "bytes")


if __name__ == "__main__":
    main()
