"""Extracts a few tensors of the GGUF files the reference tree bundles into tests/golden/gguf_tensors.npz, with
the reference's own decode and exact-tier GEMM of each (oracle/_ref/libkrk_ref.so). These are the only real
(not synthetic) quantized blocks available: Q8_0, Q5_0, Q5_1 and IQ4_NL tensors of two tiny test models.

    make -C oracle ref && KRK_REF=<kraken tree> python tests/golden/make_gguf_golden.py

The files are parsed here by a few lines of Python that know nothing of the library's reader, so that the
reader under test (krk_gguf_*) is checked against an independent parse. The tests read only the .npz.
"""
from __future__ import annotations

import os
import struct
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from kraken_b200 import synth  # noqa: E402
from oracle.krk_oracle import Reference  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("KRK_REF") or os.path.join(os.path.dirname(ROOT), "reference")
SCALAR = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}
# (file, tensor, rows kept): whole small tensors, and the first rows of the 128256-row head
PICKS = [("TinyLLama-v0.Q8_0.gguf", "blk.0.attn_q.weight", None), ("TinyLLama-v0.Q8_0.gguf", "blk.3.ffn_down.weight", None),
         ("TinyLLama-v0.Q8_0.gguf", "token_embd.weight", 512), ("tiny-llama3-test-Q3_K_M.gguf", "output.weight", 1024),
         ("tiny-llama3-test-Q3_K_M.gguf", "token_embd.weight", 1024), ("tiny-llama3-test-Q3_K_M.gguf", "*Q5_0*", None),
         ("tiny-llama3-test-Q3_K_M.gguf", "*Q5_1*", None), ("tinystories-gpt-0.1-3m.Q2_K.gguf", "*IQ4_NL*", None)]
WANT = {"*Q5_0*": 6, "*Q5_1*": 7, "*IQ4_NL*": 20}


def parse(path):
    """-> (version, {key: value or ('array', elem, count)}, [(name, dims, type, offset)], data_off)"""
    buf = open(path, "rb").read()
    pos = 0

    def take(fmt):
        nonlocal pos
        v = struct.unpack_from("<" + fmt, buf, pos)
        pos += struct.calcsize("<" + fmt)
        return v[0] if len(v) == 1 else v

    def string():
        nonlocal pos
        n = take("Q")
        s = buf[pos:pos + n].decode("utf-8", "replace")
        pos += n
        return s
    assert take("I") == 0x46554747
    version, n_tensors, n_kv = take("I"), take("Q"), take("Q")
    kvs = {}
    for _ in range(n_kv):
        key, t = string(), take("I")
        if t == 8:
            kvs[key] = string()
        elif t == 9:
            et, cnt = take("I"), take("Q")
            for _ in range(cnt):
                string() if et == 8 else take(SCALAR[et])
            kvs[key] = ("array", et, cnt)
        else:
            kvs[key] = take(SCALAR[t])
    tensors = []
    for _ in range(n_tensors):
        name, nd = string(), take("I")
        dims = [take("Q") for _ in range(nd)]
        tensors.append((name, dims, take("I"), take("Q")))
    align = int(kvs.get("general.alignment", 32))
    return version, kvs, tensors, (pos + align - 1) // align * align, buf


def main():
    ref = Reference(threads=2)
    data, files = {}, {}
    for i, (fname, pick, keep) in enumerate(PICKS):
        path = os.path.join(REF, fname)
        if fname not in files:
            files[fname] = parse(path)
            version, kvs, tensors, data_off, _ = files[fname]
            tag = f"file{len(files) - 1}"
            data[f"{tag}_name"] = np.array(fname)
            data[f"{tag}_summary"] = np.array([version, len(kvs), len(tensors), data_off], np.int64)
            data[f"{tag}_tensor_names"] = np.array([t[0] for t in tensors])
            data[f"{tag}_tensor_types"] = np.array([t[2] for t in tensors], np.int32)
            data[f"{tag}_tensor_offsets"] = np.array([t[3] for t in tensors], np.int64)
            data[f"{tag}_arch"] = np.array(kvs.get("general.architecture", ""))
        version, kvs, tensors, data_off, buf = files[fname]
        if pick in WANT:   # the first 2-d tensor of that type
            cands = [t for t in tensors if t[2] == WANT[pick] and len(t[1]) == 2]
            if not cands:
                continue
            t = cands[0]
        else:
            t = next(t for t in tensors if t[0] == pick)
        name, dims, wt, off = t
        n_in, n_rows = dims[0], dims[1]
        rows = n_rows if keep is None else min(keep, n_rows)
        rb = synth.row_bytes(wt, n_in)
        w = np.frombuffer(buf, np.uint8, rows * rb, data_off + off).reshape(rows, rb).copy()
        x = synth.activations(2, n_in, synth.BASE_SEED + 300 + i)
        key = f"t{i}"
        data[f"{key}_file"], data[f"{key}_name"] = np.array(fname), np.array(name)
        data[f"{key}_meta"] = np.array([wt, n_in, n_rows, rows, off], np.int64)
        data[f"{key}_w"], data[f"{key}_x"] = w, x
        data[f"{key}_deq"] = ref.dequant_rows(w, wt, rows, n_in)
        data[f"{key}_y"] = ref.gemm(x, w, wt, rows, n_in, rows=2, tier=0)
    out = os.path.join(OUT, "gguf_tensors.npz")
    np.savez_compressed(out, **data)
    print("wrote", out, os.path.getsize(out), "bytes;", sorted(k for k in data if k.endswith("_name") and k.startswith("t")))


if __name__ == "__main__":
    main()
