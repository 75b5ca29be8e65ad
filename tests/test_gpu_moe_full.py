"""Config 5 at its stated size (128 experts, top-8, hidden 4096, expert width 1536, 16 experts per GPU) and the
router on near-ties, through the C ABI on a B200, against the CPU checker.

The bank of 128 experts is sixteen synthetic experts repeated eight times (expert e holds the bytes of expert
e % 16): the kernels see 128 distinct matrices in device memory and the checker only ever touches the picked
ones, so the full-size case stays a matter of seconds.
"""
import numpy as np
import pytest

from kraken_b200 import synth

pytestmark = pytest.mark.gpu

SEED = synth.BASE_SEED + 500
N_EMBD, N_FF, N_EXP, K, N_DISTINCT = 4096, 1536, 128, 8, 16


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def experts():
    gate = [synth.weights(synth.Q4_K, N_FF, N_EMBD, SEED, stream=1000 + e) for e in range(N_DISTINCT)]
    up = [synth.weights(synth.Q4_K, N_FF, N_EMBD, SEED, stream=2000 + e) for e in range(N_DISTINCT)]
    down = [synth.weights(synth.Q6_K, N_EMBD, N_FF, SEED, stream=3000 + e) for e in range(N_DISTINCT)]
    return gate, up, down


@pytest.fixture(scope="module")
def bank_tensors(experts):
    gate, up, down = experts
    rep = N_EXP // N_DISTINCT
    return tuple(dev(np.stack(m)).repeat(rep, 1, 1).contiguous() for m in (gate, up, down))


def oracle_lists(experts, lo=0, hi=N_EXP):
    gate, up, down = experts
    pick = lambda mats: [mats[e % N_DISTINCT] if lo <= e < hi else None for e in range(N_EXP)]
    return pick(gate), pick(up), pick(down)


@pytest.mark.parametrize("n_tok", [1, 8])
def test_config5_full_bank_128_experts(cuda, oracle, experts, bank_tensors, n_tok):
    import torch
    g, u, d = bank_tensors
    bank = cuda.make_bank(g, u, d, synth.Q4_K, synth.Q6_K, N_EXP, 0, N_EMBD, N_FF)
    x = synth.activations(n_tok, N_EMBD, SEED + n_tok)
    logits = synth.activations(n_tok, N_EXP, SEED + n_tok, stream=7)
    ids_ref, wts_ref = oracle.route(logits, K)
    y, ids, wts = cuda.moe_ffn_routed(dev(x), dev(logits), K, bank)
    assert cuda.device_status() == 0
    assert np.array_equal(ids.cpu().numpy(), ids_ref)                      # exact, ties to the lower id
    assert np.allclose(wts.cpu().numpy(), wts_ref, rtol=2e-6, atol=1e-9)
    y_ref = oracle.moe_ffn(x, ids_ref, wts_ref, *oracle_lists(experts), synth.Q4_K, synth.Q6_K, N_EMBD, N_FF, threads=8)
    rel = np.linalg.norm(y.cpu().numpy() - y_ref) / np.linalg.norm(y_ref)
    assert rel < 2e-4, f"relative L2 error {rel:.2e}"
    # the two-call form gives the same bits
    y2 = cuda.moe_ffn(dev(x), ids, wts, bank)
    assert torch.equal(y, y2)


def test_config5_sixteen_experts_per_gpu_shards_add_up(cuda, oracle, experts, bank_tensors):
    """Eight shards of 16 experts (expert_base 0, 16, ..., 112), as eight GPUs hold them: every shard's partial
    sum against the checker's partial sum over the same experts, and the rank-ordered sum of the partials against
    the whole bank."""
    g, u, d = bank_tensors
    n_tok = 8
    x = synth.activations(n_tok, N_EMBD, SEED + 31)
    logits = synth.activations(n_tok, N_EXP, SEED + 31, stream=7)
    ids_ref, wts_ref = oracle.route(logits, K)
    xd, ld = dev(x), dev(logits)
    parts = []
    per = N_EXP // 8
    for r in range(8):
        lo = r * per
        bank = cuda.make_bank(g[lo:lo + per], u[lo:lo + per], d[lo:lo + per], synth.Q4_K, synth.Q6_K, per, lo, N_EMBD, N_FF)
        part, ids, _ = cuda.moe_ffn_routed(xd, ld, K, bank)
        assert np.array_equal(ids.cpu().numpy(), ids_ref)
        held = ((ids_ref >= lo) & (ids_ref < lo + per)).any()
        ref = oracle.moe_ffn(x, ids_ref, wts_ref, *oracle_lists(experts, lo, lo + per), synth.Q4_K, synth.Q6_K, N_EMBD, N_FF,
                             threads=8)
        got = part.cpu().numpy()
        if held:
            assert np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30) < 2e-4
        else:
            assert not got.any()                                           # an idle shard contributes zeros
        parts.append(part)
    import torch
    total = cuda.sum_parts(torch.stack(parts)).cpu().numpy()
    assert cuda.device_status() == 0
    whole = oracle.moe_ffn(x, ids_ref, wts_ref, *oracle_lists(experts), synth.Q4_K, synth.Q6_K, N_EMBD, N_FF, threads=8)
    assert np.linalg.norm(total - whole) / np.linalg.norm(whole) < 2e-4
    want = parts[0].cpu().numpy().copy()
    for r in range(1, 8):
        want += parts[r].cpu().numpy()
    assert np.array_equal(total, want)                                     # ((p0 + p1) + p2) + ... exactly


def test_router_near_ties_match_the_host(cuda, oracle):
    """10,000 rows of 128 logits in which the k-th and (k+1)-th best are one or two units in the last place
    apart (in either order of their ids), plus pairs further down the ranking: the picked ids must be the
    host's. The device ranks probabilities it computes with a correctly rounded exp, as the host's expf is in
    all but a fraction of a percent of its arguments; the test allows one row in a thousand to differ, and every
    differing row must differ only by swapping two experts whose host probabilities are equal or adjacent."""
    rng = np.random.default_rng(20251125)
    n_rows = 10000
    logits = synth.activations(n_rows, N_EXP, SEED + 77, stream=7).copy()
    order = np.argsort(-logits, axis=1, kind="stable")
    for r in range(n_rows):
        pos = K - 1 if r % 2 == 0 else int(rng.integers(0, K + 2))         # around the k-th pick, or anywhere near the top
        a, b = order[r, pos], order[r, pos + 1]
        steps = int(rng.integers(0, 3))                                    # 0: exact tie, 1 or 2 ulps apart
        v = logits[r, a]
        for _ in range(steps):
            v = np.nextafter(v, np.float32(-np.inf), dtype=np.float32)
        logits[r, b] = v
    ids_ref, wts_ref = oracle.route(logits, K)
    ids, wts = cuda.route(dev(logits), K)
    ids = ids.cpu().numpy()
    bad = np.nonzero((ids != ids_ref).any(axis=1))[0]
    assert len(bad) <= n_rows // 1000, f"{len(bad)} of {n_rows} near-tie rows picked other experts than the host"
    for r in bad:
        diff = set(ids[r].tolist()) ^ set(ids_ref[r].tolist())
        assert len(diff) <= 2, f"row {r}: more than one swap"
    good = np.ones(n_rows, dtype=bool)
    good[bad] = False
    assert np.allclose(wts.cpu().numpy()[good], wts_ref[good], rtol=2e-6, atol=1e-9)


@pytest.mark.parametrize("n_tok,n_exp,k", [(40, 16, 4), (9, 8, 2), (300, 16, 8)])
def test_moe_more_than_eight_tokens_expert_major(cuda, oracle, n_tok, n_exp, k):
    """Prefill batches: the expert-major grouped path (gather the tokens of an expert, gate / up / down on the
    tensor cores, scatter-add in ascending expert id) against the checker's per-expert loop. The GEMMs round the
    activations to f16 (the prefill bar is 2e-3 of ||w_row|| * ||x_row|| per product), so the end-to-end bar is a
    relative L2 of 3e-3; experts with at most eight tokens run the decode GEMV."""
    n_embd, n_ff = 1024, 512
    seed = SEED + 900 + n_tok
    gate = [synth.weights(synth.Q4_K, n_ff, n_embd, seed, stream=1000 + e) for e in range(n_exp)]
    up = [synth.weights(synth.Q4_K, n_ff, n_embd, seed, stream=2000 + e) for e in range(n_exp)]
    down = [synth.weights(synth.Q6_K, n_embd, n_ff, seed, stream=3000 + e) for e in range(n_exp)]
    # activations of a size that keeps silu(gate) * up inside the f16 range the GEMM stages its input in (the
    # synthetic weights are far larger than a trained model's)
    x = synth.activations(n_tok, n_embd, seed) * np.float32(0.125)
    logits = synth.activations(n_tok, n_exp, seed, stream=7)
    ids_ref, wts_ref = oracle.route(logits, k)
    y_ref = oracle.moe_ffn(x, ids_ref, wts_ref, gate, up, down, synth.Q4_K, synth.Q6_K, n_embd, n_ff, threads=8)
    bank = cuda.make_bank(dev(np.stack(gate)), dev(np.stack(up)), dev(np.stack(down)), synth.Q4_K, synth.Q6_K, n_exp, 0,
                          n_embd, n_ff)
    y, ids, wts = cuda.moe_ffn_routed(dev(x), dev(logits), k, bank)
    assert cuda.device_status() == 0
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    rel = np.linalg.norm(y.cpu().numpy() - y_ref) / np.linalg.norm(y_ref)
    assert rel < 3e-3, f"relative L2 error {rel:.2e}"
    # a shard (the upper half of the experts) gives the checker's partial sum over those experts
    lo = n_exp // 2
    part_bank = cuda.make_bank(dev(np.stack(gate[lo:])), dev(np.stack(up[lo:])), dev(np.stack(down[lo:])), synth.Q4_K,
                               synth.Q6_K, n_exp - lo, lo, n_embd, n_ff)
    part = cuda.moe_ffn(dev(x), ids, wts, part_bank).cpu().numpy()
    sel = lambda mats: [m if e >= lo else None for e, m in enumerate(mats)]
    part_ref = oracle.moe_ffn(x, ids_ref, wts_ref, sel(gate), sel(up), sel(down), synth.Q4_K, synth.Q6_K, n_embd, n_ff, threads=8)
    assert np.linalg.norm(part - part_ref) / np.linalg.norm(part_ref) < 3e-3


def test_router_steps_and_plan_match_the_host(cuda, oracle):
    """router_softmax -> router_topk -> moe_plan_build, the three steps of the Backend interface: ids and weights
    are the one-call router's (hence the host's), the plan is the host's expert-major plan (tokens ascending, then
    slots ascending, within each expert)."""
    n_tok, n_exp, k = 37, 128, 8
    logits = synth.activations(n_tok, n_exp, SEED + 41, stream=7)
    ld = dev(logits)
    probs = cuda.router_softmax(ld)
    ids, wts = cuda.router_topk(probs, k)
    ids1, wts1 = cuda.route(ld, k)
    import torch
    assert torch.equal(ids, ids1) and torch.equal(wts, wts1)
    ids_ref, wts_ref = oracle.route(logits, k)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    p = probs.cpu().numpy()
    assert np.allclose(p.sum(axis=1), 1.0, atol=1e-5)
    _, raw = cuda.router_topk(probs, k, normalize=False, scale=2.0)
    picked = np.take_along_axis(p, ids_ref.astype(np.int64), axis=1)
    assert np.array_equal(raw.cpu().numpy(), (picked * np.float32(2.0)).astype(np.float32))
    off, rows, wt = (t.cpu().numpy() for t in cuda.moe_plan_build(ids, wts, n_exp))
    want_off, want_rows, want_wt = [0], [], []
    w_np = wts.cpu().numpy()
    for e in range(n_exp):
        for t in range(n_tok):
            for s in range(k):
                if ids_ref[t, s] == e:
                    want_rows.append(t)
                    want_wt.append(w_np[t, s])
        want_off.append(len(want_rows))
    assert off.tolist() == want_off and rows.tolist() == want_rows and wt.tolist() == want_wt
