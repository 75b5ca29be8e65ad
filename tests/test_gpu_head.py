"""The steps either side of the output head on the device: embedding gather (bit-exact with the host
decoders, zero rows for bad ids) and top-k of a logits row (ids and values exactly those of the
reference's CPU twin, ties toward the lower id, mass within f32 summation-order noise)."""
import numpy as np
import pytest

from kraken_b200 import synth

pytestmark = pytest.mark.gpu
SEED = synth.BASE_SEED + 31


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("wt", [synth.Q8_0, synth.Q4_0, synth.Q4_K, synth.Q6_K])
def test_embed_bit_exact(cuda, oracle, golden, wt):
    name = synth.NAMES[wt].lower()
    table, toks = golden[f"embed_{name}_table"], golden[f"embed_{name}_tokens"]
    got = cuda.embed(dev(table), wt, 40, 512, dev(toks)).cpu().numpy()
    assert got.tobytes() == golden[f"embed_{name}_out"].tobytes()
    # a bigger table, random-byte payload, ids at both ends and outside
    n_vocab, n_embd = 1000, 2048
    table = synth.weights(wt, n_vocab, n_embd, SEED, stream=wt, random_payload=True)
    toks = np.array([0, 999, 1000, -1, 512, 7, 7, 2**31 - 1], np.int32)
    got = cuda.embed(dev(table), wt, n_vocab, n_embd, dev(toks)).cpu().numpy()
    want = oracle.embed(table, wt, n_vocab, n_embd, toks)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(np.nan_to_num(got).view(np.uint32), np.nan_to_num(want).view(np.uint32))
    assert cuda.device_status() == 0


def keys_f32(lg, pm, pen, cap):
    """The reference's key (src/backend_cpu.cpp:872-881) over a whole row, in f32."""
    v = lg.astype(np.float32).copy()
    if cap > 0.0:
        v = np.clip(v, np.float32(-cap), np.float32(cap))
    if pm is not None and pen > 0.0 and pen != 1.0:
        i = np.arange(v.size, dtype=np.uint32)
        hit = ((pm[i >> 5] >> (i & 31)) & 1).astype(bool)
        v = np.where(hit, np.where(v > 0, v / np.float32(pen), v * np.float32(pen)), v).astype(np.float32)
    return v


def check_topk(cuda, oracle, lg, k, pm=None, pen=1.0, cap=0.0, temp=1.0):
    ids, vals, mass = cuda.logits_topk(dev(lg), k, None if pm is None else dev(pm), pen, cap, temp)
    ids_ref, vals_ref, mass_ref = oracle.logits_topk(lg, k, pm, pen, cap, temp)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    assert vals.cpu().numpy().tobytes() == vals_ref.tobytes()
    # mass: the reference adds the row's exponentials one after another in f32, which over 128256 terms
    # drifts by ~1e-4 relative; the device adds per slice. Tight against the f64 sum, loose against the
    # reference's own f32 chain.
    key = keys_f32(lg, pm, pen, cap).astype(np.float64)
    exact = float(np.exp((key - key.max()) / (temp if temp > 0 else 1.0)).sum())
    assert abs(float(mass.item()) - exact) <= 2e-5 * exact, (float(mass.item()), exact)
    assert abs(float(mass.item()) - mass_ref) <= 1e-3 * abs(mass_ref), (float(mass.item()), mass_ref)


def test_topk_reference_vectors(cuda, oracle, golden):
    lg, pm = golden["topk_logits"], golden["topk_mask"]
    for tag in "abc":
        k, cap, pen, temp = golden[f"topk_{tag}_args"]
        ids, vals, mass = cuda.logits_topk(dev(lg), int(k), dev(pm), float(pen), float(cap), float(temp))
        assert np.array_equal(ids.cpu().numpy(), golden[f"topk_{tag}_ids"])
        assert vals.cpu().numpy().tobytes() == golden[f"topk_{tag}_vals"].tobytes()
        assert abs(float(mass.item()) - float(golden[f"topk_{tag}_mass"])) <= 2e-5 * float(golden[f"topk_{tag}_mass"])
    ids, vals, _ = cuda.logits_topk(dev(lg[:5]), 8)
    assert np.array_equal(ids.cpu().numpy(), golden["topk_short_ids"])
    assert vals.cpu().numpy().tobytes() == golden["topk_short_vals"].tobytes()


def test_topk_full_vocabulary_ties_and_edges(cuda, oracle):
    n = 128256                                            # config 4's row
    lg = synth.normal(n, SEED, 5) * 3.0
    lg[77] = lg[100000] = lg[128255] = lg.max() + 2.0     # a three-way tie across slices: ids ascending
    lg[5:9] = lg[5]                                       # a tie inside one slice
    pm = np.zeros((n + 31) // 32, np.uint32)
    pm[::7] = 0x80000001
    check_topk(cuda, oracle, lg, 1)
    check_topk(cuda, oracle, lg, 40, pm, 1.2, 30.0, 0.8)
    check_topk(cuda, oracle, lg, 64, pm, 0.9, 4.0, 1.0)    # softcap makes thousands of keys equal: order by id
    same = np.full(4100, 0.25, np.float32)                # everything ties
    check_topk(cuda, oracle, same, 8)
    tiny = np.array([1.0, -np.inf, 3.0], np.float32)      # fewer than k, one of them -inf
    ids, vals, _ = cuda.logits_topk(dev(tiny), 4)
    assert ids.cpu().tolist() == [2, 0, 1, -1]
    assert vals.cpu().tolist()[3] == float(np.finfo(np.float32).min)
    assert cuda.device_status() == 0


def test_head_then_topk_equals_host_argmax(cuda, oracle):
    """An eighth of config 4's head, the logits stay on the device: top-1 = argmax of the oracle's logits."""
    import torch
    n_out, n_in = 128256 // 8, 4096
    w = synth.weights(synth.Q6_K, n_out, n_in, SEED + 4, stream=synth.Q6_K)
    x = synth.activations(1, n_in, SEED + 4)
    logits = cuda.gemv(dev(x), dev(w), synth.Q6_K, n_out, n_in)
    ids, vals, _ = cuda.logits_topk(logits.reshape(-1), 5)
    ref = oracle.gemm(x, w, synth.Q6_K, n_out, n_in, rows=1, threads=8).reshape(-1)
    order = np.argsort(-ref, kind="stable")[:5]
    gaps = ref[order[:-1]] - ref[order[1:]]
    if gaps.min() > 1e-3 * np.abs(ref).max():             # well separated: the ranking must agree exactly
        assert ids.cpu().tolist() == order.tolist()
    assert ids.cpu().tolist()[0] == int(order[0]) or abs(ref[ids.cpu().tolist()[0]] - ref[order[0]]) < 1e-3 * np.abs(ref).max()


def test_head_refusals(cuda):
    import torch
    from kraken_b200 import capi
    lg = torch.zeros(100, device="cuda")
    ids = torch.zeros(4, dtype=torch.int32, device="cuda")
    vals = torch.zeros(4, device="cuda")
    ws = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    L = capi.lib                                          # codes: EDTYPE -1, ESHAPE -2, EWORKSPACE -6, EARG -8
    assert L.krk_cuda_logits_topk(lg.data_ptr(), 100, 0, None, 1.0, 0.0, 1.0, ids.data_ptr(), vals.data_ptr(), None,
                                  ws.data_ptr(), 4096, None) == -8
    assert L.krk_cuda_logits_topk(lg.data_ptr(), 100, 65, None, 1.0, 0.0, 1.0, ids.data_ptr(), vals.data_ptr(), None,
                                  ws.data_ptr(), 4096, None) == -8
    assert L.krk_cuda_logits_topk(lg.data_ptr(), 100, 4, None, 1.0, 0.0, 1.0, ids.data_ptr(), vals.data_ptr(), None,
                                  ws.data_ptr(), 8, None) == -6
    assert L.krk_cuda_embed(vals.data_ptr(), ws.data_ptr(), 99, 10, 256, ids.data_ptr(), 1, None) == -1
    assert L.krk_cuda_embed(vals.data_ptr(), ws.data_ptr(), synth.Q4_K, 10, 100, ids.data_ptr(), 1, None) == -2
