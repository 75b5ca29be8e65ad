"""The CPU checker against the reference's golden vectors (no GPU)."""
import numpy as np
import pytest

from kraken_b200 import synth

FMTS = [synth.Q8_0, synth.Q4_0, synth.Q4_K, synth.Q6_K]


def test_geometry(oracle):
    # the reference suite's own geometry pins (tests/test_kraken.cpp:396-403)
    assert oracle.block_size(synth.Q4_0) == 32 and oracle.block_bytes(synth.Q4_0) == 18
    assert oracle.block_size(synth.Q6_K) == 256 and oracle.block_bytes(synth.Q6_K) == 210
    assert oracle.row_bytes(synth.Q8_0, 64) == 68
    assert oracle.block_bytes(synth.Q4_K) == 144 and oracle.block_bytes(synth.Q8_0) == 34
    assert oracle.block_size(99) == 0 and oracle.row_bytes(99, 64) == 0
    for wt in FMTS:
        assert oracle.row_bytes(wt, 4096) == synth.row_bytes(wt, 4096)


def test_fp16_table(oracle, golden):
    got = np.array([oracle.fp16_to_fp32(h) for h in range(65536)], np.float32).view(np.uint32)
    assert (got == golden["fp16_table"]).all()


@pytest.mark.parametrize("wt", FMTS)
@pytest.mark.parametrize("tag", ["field", "bytes"])
def test_decode_and_gemm_match_reference_vectors(oracle, golden, wt, tag):
    name = synth.NAMES[wt].lower()
    w, x = golden[f"{name}_{tag}_w"], golden[f"{name}_{tag}_x"]
    n_rows, n_in = w.shape[0], x.shape[1]
    deq = oracle.dequant_rows(w, wt, n_rows, n_in)
    assert deq.tobytes() == golden[f"{name}_{tag}_deq"].tobytes()          # bit-exact
    for threads in (1, 3):
        y = oracle.gemm(x, w, wt, n_rows, n_in, rows=x.shape[0], threads=threads)
        assert y.tobytes() == golden[f"{name}_{tag}_y"].tobytes()          # bit-exact, any thread count


def test_known_answer_blocks(oracle, golden):
    # tests/test_kraken.cpp:456-469: d=1, nibbles i|i<<4 -> i-8 twice
    q40 = oracle.dequant_rows(golden["kat_q4_0_w"], synth.Q4_0, 1, 32)[0]
    assert np.array_equal(q40[:16], np.arange(16) - 8.0) and np.array_equal(q40[16:], np.arange(16) - 8.0)
    # :563-573: d=0.5, q=i-16
    q80 = oracle.dequant_rows(golden["kat_q8_0_w"], synth.Q8_0, 1, 32)[0]
    assert np.array_equal(q80, 0.5 * (np.arange(32) - 16.0))
    # :981-1001: bounded sum; with every 6-bit field = 1 the value is 0.5*1*8 - 0.25*1 = 3.75
    q4k = oracle.dequant_rows(golden["kat_q4_k_w"], synth.Q4_K, 1, 256)[0]
    assert abs(q4k.sum()) < 256.0 * 8.0
    # :1026-1042: qh advances 32 bytes per 128-value half
    q6k = oracle.dequant_rows(golden["kat_q6_k_w"], synth.Q6_K, 1, 256)[0]
    assert q6k[0] == -32.0 and q6k[128] == 16.0 and q6k[160] == -32.0
    for key, wt, n in (("kat_q4_0", synth.Q4_0, 32), ("kat_q8_0", synth.Q8_0, 32),
                       ("kat_q4_k", synth.Q4_K, 256), ("kat_q6_k", synth.Q6_K, 256)):
        assert oracle.dequant_rows(golden[f"{key}_w"], wt, 1, n).tobytes() == golden[f"{key}_deq"].tobytes()


def test_silu_and_scatter(oracle, golden):
    assert oracle.silu_mul(golden["silu_gate"], golden["silu_up"]).tobytes() == golden["silu_out"].tobytes()
    dst = golden["scatter_dst"].copy()
    oracle.scatter_axpy_rows(dst, golden["scatter_src"], golden["scatter_rows"], golden["scatter_alpha"])
    assert dst.tobytes() == golden["scatter_out"].tobytes()


def test_embed_and_topk_match_reference_vectors(oracle, golden):
    for wt in FMTS:
        name = synth.NAMES[wt].lower()
        out = oracle.embed(golden[f"embed_{name}_table"], wt, 40, 512, golden[f"embed_{name}_tokens"])
        assert out.tobytes() == golden[f"embed_{name}_out"].tobytes()
        assert not out[2].any() and not out[3].any()                    # ids -1 and 40: zero rows
    lg, pm = golden["topk_logits"], golden["topk_mask"]
    for tag in "abc":
        k, cap, pen, temp = golden[f"topk_{tag}_args"]
        ids, vals, mass = oracle.logits_topk(lg, int(k), pm, float(pen), float(cap), float(temp))
        assert np.array_equal(ids, golden[f"topk_{tag}_ids"])
        assert vals.tobytes() == golden[f"topk_{tag}_vals"].tobytes()
        assert np.float32(mass) == golden[f"topk_{tag}_mass"]
    assert golden["topk_a_ids"][0] == 100                               # the tie goes to the lower id
    ids, vals, _ = oracle.logits_topk(lg[:5], 8)
    assert np.array_equal(ids, golden["topk_short_ids"]) and ids[5] == -1
    assert vals.tobytes() == golden["topk_short_vals"].tobytes()


def test_refusals(oracle):
    w = np.zeros(144, np.uint8)
    with pytest.raises(ValueError):
        oracle.dequant_rows(w, synth.Q4_K, 1, 100)      # not a whole super-block
    with pytest.raises(ValueError):
        oracle.dequant_rows(w, 99, 1, 256)              # unknown type
    with pytest.raises(ValueError):
        oracle.gemm(np.zeros(100, np.float32), w, synth.Q4_K, 1, 100)
    assert oracle.gemm(np.zeros((0, 256), np.float32), w, synth.Q4_K, 1, 256, rows=0).shape == (0, 1)
    assert oracle.gemm(np.zeros((1, 256), np.float32), w[:0], synth.Q4_K, 0, 256).shape == (1, 0)


def test_route_rules(oracle):
    # softmax -> top-k with ties to the lower id -> renormalise over the picks
    logits = np.zeros((2, 16), np.float32)
    logits[0, [3, 9, 12]] = [2.0, 2.0, 1.0]            # tie between 3 and 9: 3 first
    logits[1] = np.arange(16)[::-1]
    ids, wts = oracle.route(logits, 4)
    assert ids[0].tolist()[:3] == [3, 9, 12] and ids[0, 3] == 0     # remaining tie at 0.0 -> id 0
    assert ids[1].tolist() == [0, 1, 2, 3]
    assert np.allclose(wts.sum(axis=1), 1.0, atol=1e-6)
    p = np.exp(logits[1] - logits[1].max()); p /= p.sum()
    assert np.allclose(wts[1], p[:4] / p[:4].sum(), rtol=1e-5)


def test_moe_composition_matches_stepwise(oracle):
    """One-expert MoE == dense FFN, and shards sum to the whole (cf. tests/test_kraken.cpp:15328)."""
    n_embd, n_ff, n_exp, k, n_tok = 256, 512, 6, 2, 3
    seed = synth.BASE_SEED + 5
    gate = [synth.weights(synth.Q4_K, n_ff, n_embd, seed, stream=10 + e) for e in range(n_exp)]
    up = [synth.weights(synth.Q4_K, n_ff, n_embd, seed, stream=30 + e) for e in range(n_exp)]
    down = [synth.weights(synth.Q6_K, n_embd, n_ff, seed, stream=50 + e) for e in range(n_exp)]
    x = synth.activations(n_tok, n_embd, seed)
    ids, wts = oracle.route(synth.activations(n_tok, n_exp, seed, stream=7), k)
    y = oracle.moe_ffn(x, ids, wts, gate, up, down, synth.Q4_K, synth.Q6_K, n_embd, n_ff)
    # step by step, ascending expert id
    want = np.zeros_like(y)
    for e in range(n_exp):
        for t in range(n_tok):
            for s in range(k):
                if ids[t, s] != e:
                    continue
                g = oracle.gemm(x[t], gate[e], synth.Q4_K, n_ff, n_embd)
                u = oracle.gemm(x[t], up[e], synth.Q4_K, n_ff, n_embd)
                d = oracle.gemm(oracle.silu_mul(g, u), down[e], synth.Q6_K, n_embd, n_ff)
                want[t] += wts[t, s] * d[0]
    assert y.tobytes() == want.tobytes()
    # two shards of the bank: partials add up to the whole within f32 rounding
    lo = [m if e < 3 else None for e, m in enumerate(gate)], [m if e < 3 else None for e, m in enumerate(up)], \
         [m if e < 3 else None for e, m in enumerate(down)]
    hi = [m if e >= 3 else None for e, m in enumerate(gate)], [m if e >= 3 else None for e, m in enumerate(up)], \
         [m if e >= 3 else None for e, m in enumerate(down)]
    y0 = oracle.moe_ffn(x, ids, wts, *lo, synth.Q4_K, synth.Q6_K, n_embd, n_ff)
    y1 = oracle.moe_ffn(x, ids, wts, *hi, synth.Q4_K, synth.Q6_K, n_embd, n_ff)
    assert np.allclose(y0 + y1, y, rtol=1e-5, atol=1e-5 * np.abs(y).max())


@pytest.mark.parametrize("wt", FMTS)
def test_oracle_equals_compiled_reference_live(oracle, reference, wt):
    """Fresh random blocks (all payload bytes random), restatement vs the reference's own code."""
    n_rows, n_in = 33, 2048
    w = synth.weights(wt, n_rows, n_in, seed=20261125, stream=wt, random_payload=True)
    x = synth.activations(2, n_in, seed=20261125)
    assert oracle.dequant_rows(w, wt, n_rows, n_in).tobytes() == reference.dequant_rows(w, wt, n_rows, n_in).tobytes()
    assert oracle.gemm(x, w, wt, n_rows, n_in, rows=2).tobytes() == \
        reference.gemm(x, w, wt, n_rows, n_in, rows=2, tier=0).tobytes()
    assert np.float32(reference.vec_dot(wt, w[0], x[0])) == oracle.gemm(x[0], w[:1], wt, 1, n_in)[0, 0]
    toks = np.array([0, 32, 7, 33, -5], np.int32)
    assert oracle.embed(w, wt, n_rows, n_in, toks).tobytes() == reference.embed(w, wt, n_rows, n_in, toks).tobytes()
    lg = synth.normal(3000, 20261125, 40 + wt) * 3.0
    a, b = oracle.logits_topk(lg, 16, None, 1.0, 2.5, 0.8), reference.logits_topk(lg, 16, None, 1.0, 2.5, 0.8)
    assert np.array_equal(a[0], b[0]) and a[1].tobytes() == b[1].tobytes() and a[2] == b[2]
