"""The GGUF tensor reader (krk_gguf_*, kraken_b200/csrc/krk_gguf.cpp): a file written by this test with every
value type the format has, the real files of the reference tree where it is mounted (against an independent
parse kept in tests/golden/gguf_tensors.npz), malformed files, and - on a GPU - the real quantized tensors of
those files through upload, decode and GEMV against the reference's own results."""
import os
import struct

import numpy as np
import pytest

from kraken_b200 import capi, synth
from tests.conftest import bound_ok

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden", "gguf_tensors.npz")


def gguf_string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, kvs, tensors, version=3, alignment=32):
    """kvs: [(key, type_id, value)]; tensors: [(name, dims, type_id, bytes)] (GGUF: dims[0] is the row length)."""
    fmt = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "?", 10: "Q", 11: "q", 12: "d"}
    out = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kvs))
    for key, t, v in kvs:
        out += gguf_string(key) + struct.pack("<I", t)
        if t == 8:
            out += gguf_string(v)
        elif t == 9:
            et, items = v
            out += struct.pack("<IQ", et, len(items))
            for it in items:
                out += gguf_string(it) if et == 8 else struct.pack("<" + fmt[et], it)
        else:
            out += struct.pack("<" + fmt[t], v)
    offsets, pos = [], 0
    for _, _, _, payload in tensors:
        offsets.append(pos)
        pos += (len(payload) + alignment - 1) // alignment * alignment
    for (name, dims, t, _), off in zip(tensors, offsets):
        out += gguf_string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", t, off)
    out += b"\0" * ((-len(out)) % alignment)
    for (_, _, _, payload), off in zip(tensors, offsets):
        pad = (-len(payload)) % alignment
        out += payload + b"\0" * pad
    open(path, "wb").write(out)


def test_reader_on_a_file_with_every_value_type(tmp_path):
    seed = synth.BASE_SEED + 600
    w8 = synth.weights(synth.Q8_0, 7, 96, seed, stream=1)
    w4 = synth.weights(synth.Q4_K, 5, 512, seed, stream=2)
    f32 = np.arange(12, dtype=np.float32)
    kvs = [("general.architecture", 8, "llama"), ("general.alignment", 4, 64), ("a.u8", 0, 200), ("a.i8", 1, -3),
           ("a.u16", 2, 65000), ("a.i16", 3, -300), ("a.i32", 5, -70000), ("a.f32", 6, 1.5), ("a.bool", 7, True),
           ("a.u64", 10, 2 ** 40), ("a.i64", 11, -(2 ** 40)), ("a.f64", 12, 2.25), ("tokenizer.tokens", 9, (8, ["a", "bc", ""])),
           ("a.ints", 9, (5, [1, -2, 3]))]
    tensors = [("blk.0.q.weight", [96, 7], synth.Q8_0, w8.tobytes()), ("blk.0.up.weight", [512, 5], synth.Q4_K, w4.tobytes()),
               ("norm.weight", [12], 0, f32.tobytes()), ("odd.weight", [256, 2], 16, b"\1" * 132)]   # type 16: not sized here
    path = str(tmp_path / "t.gguf")
    write_gguf(path, kvs, tensors, alignment=64)
    g = capi.Gguf(path)
    assert g.version == 3 and len(g) == 4 and g.kv_count() == len(kvs)
    assert g.get_str("general.architecture") == "llama" and g.get_int("general.alignment") == 64
    assert g.get_int("a.u8") == 200 and g.get_int("a.i8") == -3 and g.get_int("a.u16") == 65000 and g.get_int("a.i16") == -300
    assert g.get_int("a.i32") == -70000 and g.get_float("a.f32") == 1.5 and g.get_int("a.bool") == 1
    assert g.get_int("a.u64") == 2 ** 40 and g.get_int("a.i64") == -(2 ** 40) and g.get_float("a.f64") == 2.25
    assert g.array_count("tokenizer.tokens") == (3, 8) and g.array_count("a.ints") == (3, 5)
    assert g.get_int("missing") is None and g.get_str("a.u8") is None and g.find("nope") == -1
    t = g.info(g.find("blk.0.q.weight"))
    assert (t.type_id, t.supported, t.n_dims, t.ne[0], t.ne[1], t.n_bytes) == (synth.Q8_0, 1, 2, 96, 7, w8.nbytes)
    assert g.tensor_bytes(0).tobytes() == w8.tobytes() and g.tensor_bytes(1).tobytes() == w4.tobytes()
    assert g.tensor_bytes(2).view(np.float32).tolist() == f32.tolist()
    t = g.info(3)
    assert t.supported == 0 and t.n_bytes == 0 and t.type_id == 16
    g.close()
    write_gguf(path, kvs[:1], tensors[:1], version=2)                     # the older version parses the same way
    g = capi.Gguf(path)
    assert g.version == 2 and g.tensor_bytes(0).tobytes() == w8.tobytes()
    g.close()


def test_reader_refuses_malformed_files(tmp_path):
    good = str(tmp_path / "good.gguf")
    write_gguf(good, [("general.architecture", 8, "x")], [("w", [32, 2], synth.Q8_0, b"\0" * 68)])
    raw = open(good, "rb").read()
    cases = {"bad magic": b"GGUX" + raw[4:], "version 9": raw[:4] + struct.pack("<I", 9) + raw[8:],
             "truncated directory": raw[:40], "data past the end": raw[:-40], "empty": b""}
    for what, payload in cases.items():
        p = str(tmp_path / "bad.gguf")
        open(p, "wb").write(payload)
        with pytest.raises(ValueError):
            capi.Gguf(p)
    with pytest.raises(ValueError):
        capi.Gguf(str(tmp_path / "absent.gguf"))
    # headers that ask for more than the file can hold: a tensor count beyond the file's size, a shape whose byte
    # count wraps around 64 bits, an alignment of 2^40
    p = str(tmp_path / "bad.gguf")
    open(p, "wb").write(raw[:8] + struct.pack("<Q", 1 << 23) + raw[16:])
    with pytest.raises(ValueError):
        capi.Gguf(p)
    write_gguf(p, [], [("w", [32, 1 << 40, 1 << 40], synth.Q8_0, b"\0" * 68)])
    with pytest.raises(ValueError):
        capi.Gguf(p)
    write_gguf(p, [("general.alignment", 10, 1 << 40)], [("w", [32, 2], synth.Q8_0, b"\0" * 68)], alignment=32)
    with pytest.raises(ValueError):
        capi.Gguf(p)


def reference_file(name):
    ref = os.environ.get("KRK_REF") or os.path.join(os.path.dirname(ROOT), "reference")
    p = os.path.join(ref, name)
    return p if os.path.exists(p) else None


def test_reader_on_the_reference_fixtures_matches_an_independent_parse():
    gold = np.load(GOLD)
    seen = 0
    for i in range(3):
        if f"file{i}_name" not in gold.files:
            continue
        path = reference_file(str(gold[f"file{i}_name"]))
        if path is None:
            continue
        seen += 1
        g = capi.Gguf(path)
        version, n_kv, n_tensors, _ = gold[f"file{i}_summary"].tolist()
        assert (g.version, g.kv_count(), len(g)) == (version, n_kv, n_tensors)
        assert g.get_str("general.architecture") == str(gold[f"file{i}_arch"])
        names, types = gold[f"file{i}_tensor_names"], gold[f"file{i}_tensor_types"]
        for j in range(n_tensors):
            t = g.info(j)
            assert t.name.decode() == str(names[j]) and t.type_id == int(types[j])
        for key in [k[:-5] for k in gold.files if k.endswith("_file") and str(gold[k]) == str(gold[f"file{i}_name"])]:
            wt, n_in, n_rows, rows, _ = gold[f"{key}_meta"].tolist()
            idx = g.find(str(gold[f"{key}_name"]))
            t = g.info(idx)
            assert (t.type_id, t.ne[0], t.ne[1]) == (wt, n_in, n_rows) and t.n_bytes == n_rows * synth.row_bytes(wt, n_in)
            assert g.tensor_bytes(idx)[:rows * synth.row_bytes(wt, n_in)].tobytes() == gold[f"{key}_w"].tobytes()
        g.close()
    if seen == 0:
        pytest.skip("the reference tree is not mounted here")


def test_oracle_on_real_tensors_matches_the_reference(oracle):
    gold = np.load(GOLD)
    keys = sorted(k[:-5] for k in gold.files if k.endswith("_meta"))
    assert len(keys) >= 6
    for key in keys:
        wt, n_in, _, rows, _ = gold[f"{key}_meta"].tolist()
        w, x = gold[f"{key}_w"], gold[f"{key}_x"]
        assert oracle.dequant_rows(w, wt, rows, n_in).tobytes() == gold[f"{key}_deq"].tobytes(), key
        assert oracle.gemm(x, w, wt, rows, n_in, rows=2, threads=4).tobytes() == gold[f"{key}_y"].tobytes(), key


@pytest.mark.gpu
def test_real_tensors_upload_decode_and_gemv(cuda, tmp_path):
    """The real blocks, written back into a GGUF file, read by the library's reader, uploaded through
    CudaBackend::upload as they lie in the file, decoded and multiplied: decode bit-exact with the reference's
    krk::dequant_row, GEMV within 1e-4 * ||w_row|| * ||x|| of its exact scalar tier."""
    import torch
    gold = np.load(GOLD)
    keys = sorted(k[:-5] for k in gold.files if k.endswith("_meta"))
    tensors = []
    for key in keys:
        wt, n_in, _, rows, _ = gold[f"{key}_meta"].tolist()
        tensors.append((key, [n_in, rows], wt, gold[f"{key}_w"].tobytes()))
    path = str(tmp_path / "real.gguf")
    write_gguf(path, [("general.architecture", 8, "llama")], tensors)
    g = cuda.Gguf(path)
    be = cuda.Backend(0)
    for key in keys:
        wt, n_in, _, rows, _ = gold[f"{key}_meta"].tolist()
        idx = g.find(key)
        d_w = g.upload(idx, be)
        nbytes = g.info(idx).n_bytes

        class View:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (d_w, False), "version": 2}
        w_dev = torch.as_tensor(View(), device="cuda")
        got = cuda.dequant_rows(w_dev, wt, rows, n_in).cpu().numpy()
        assert got.tobytes() == gold[f"{key}_deq"].tobytes(), key
        x = gold[f"{key}_x"]
        y = cuda.gemv(torch.from_numpy(x).cuda(), w_dev, wt, rows, n_in).cpu().numpy()
        ok, worst = bound_ok(y, gold[f"{key}_y"], gold[f"{key}_deq"], x, 1e-4)
        assert ok, (key, worst)
        del w_dev
        be.release(d_w)
    be.close()
    g.close()
    assert cuda.device_status() == 0
