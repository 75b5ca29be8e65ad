"""A seeded random sweep over shapes, formats and call forms of the matmul path against the CPU checker: the decode
GEMV (1..8 activation rows, K any whole number of blocks), the prefill GEMM (9..300 rows, f16 or f32 activations),
grouped launches (mixed weight types, shared or per-matrix activations, gate/up pairs with the silu fold), the
accumulating form, and the routed-expert FFN over banks of every streaming format. The single-case tests pin
named shapes; this one walks the corners between them (ragged row counts, K = 256 .. 5120, 1-row matrices)."""
import random

import numpy as np
import pytest

from conftest import bound_ok
from kraken_b200 import synth

pytestmark = pytest.mark.gpu

FMTS = list(synth.FORMATS) + list(synth.MORE_FORMATS)
K_QUANTS = (synth.Q4_K, synth.Q6_K, synth.Q5_K, synth.Q2_K, synth.Q3_K)


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def finite_rows(y, ref, w_deq, x, tol):
    """Random payloads can hold non-finite scales: those weight rows must be non-finite on both sides, the others
    within the bound."""
    fin = np.isfinite(w_deq).all(axis=1)
    ok, worst = bound_ok(y[:, fin], ref[:, fin], w_deq[fin], x, tol)
    return ok and np.array_equal(np.isfinite(y[:, ~fin]), np.isfinite(ref[:, ~fin])), worst


def test_random_gemv_and_gemm_shapes(cuda, oracle):
    rng = random.Random(20240607)
    for case in range(160):
        wt = rng.choice(FMTS)
        bs = 256 if wt in K_QUANTS else 32
        n_in = 256 * rng.randint(1, 20) if rng.random() < 0.7 else bs * rng.randint(1, 40)
        n_out = rng.choice([1, 7, 16, 17, 33, 100, 255, 513, 1000, 2049, rng.randint(1, 3000)])
        prefill = case % 3 == 2
        rows = rng.choice([9, 16, 40, 129, 257, 300]) if prefill else rng.randint(1, 8)
        seed = rng.randint(0, 1 << 30)
        w = synth.weights(wt, n_out, n_in, seed, stream=wt, random_payload=rng.random() < 0.5)
        x = synth.activations(rows, n_in, seed + 1)
        tol = 1e-4
        if prefill:
            use16 = n_in % 256 == 0 and rng.random() < 0.7
            xin = x.astype(np.float16) if use16 else x
            x = xin.astype(np.float32)
            y = cuda.gemm(dev(xin), dev(w), wt, n_out, n_in).cpu().numpy()
            tol = 2e-3 if n_in % 256 == 0 else 1e-4
        else:
            y = cuda.gemv(dev(x), dev(w), wt, n_out, n_in).cpu().numpy()
        ref = oracle.gemm(x, w, wt, n_out, n_in, rows=rows, threads=8)
        ok, worst = finite_rows(y, ref, oracle.dequant_rows(w, wt, n_out, n_in), x, tol)
        assert ok, (case, synth.NAMES[wt], n_out, n_in, rows, seed, worst)
        assert cuda.device_status() == 0


def test_random_groups_pairs_accumulate_and_experts(cuda, oracle):
    rng = random.Random(777)
    g = lambda x, w, wt, n, k, rows=1: oracle.gemm(x, w, wt, n, k, rows=rows, threads=4)
    for case in range(80):
        seed = rng.randint(0, 1 << 30)
        n_in = 256 * rng.randint(1, 12)
        kind = ("group", "pair", "acc", "moe")[case % 4]
        if kind == "group":
            n_mat = rng.randint(1, 16)
            wts = [rng.choice(FMTS) for _ in range(n_mat)] if rng.random() < 0.5 else [rng.choice(FMTS)] * n_mat
            n_outs = [rng.choice([1, 16, 33, 256, 777, 1024]) for _ in range(n_mat)]
            ws = [synth.weights(wt, no, n_in, seed, stream=10 + i) for i, (wt, no) in enumerate(zip(wts, n_outs))]
            shared = rng.random() < 0.5
            xs = [synth.activations(1, n_in, seed, stream=50 + (0 if shared else i)) for i in range(n_mat)]
            dx = [dev(x) for x in xs]
            if shared:
                dx = [dx[0]] * n_mat
            ys = cuda.gemv_group(dx, [dev(w) for w in ws], wts, n_outs, n_in)
            for i in range(n_mat):
                ok, worst = bound_ok(ys[i].cpu().numpy().reshape(1, -1), g(xs[i], ws[i], wts[i], n_outs[i], n_in),
                                     oracle.dequant_rows(ws[i], wts[i], n_outs[i], n_in), xs[i], 1e-4)
                assert ok, (case, wts, n_outs, n_in, seed, i, worst)
        elif kind == "pair":
            wt, no, pairs = rng.choice(FMTS), rng.choice([16, 100, 768, 1536]), rng.randint(1, 4)
            ws = [synth.weights(wt, no, n_in, seed, stream=10 + i) for i in range(2 * pairs)]
            xs = [synth.activations(1, n_in, seed, stream=50 + i) for i in range(pairs)]
            dxs = [dev(x) for x in xs]
            ys = cuda.gemv_group([dxs[i // 2] for i in range(2 * pairs)], [dev(w) for w in ws], [wt] * (2 * pairs),
                                 [no] * (2 * pairs), n_in, fuse_silu_pair=True)
            for i in range(pairs):
                ref = oracle.silu_mul(g(xs[i], ws[2 * i], wt, no, n_in)[0], g(xs[i], ws[2 * i + 1], wt, no, n_in)[0])
                got = ys[2 * i].cpu().numpy().reshape(-1)
                rel = np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)
                assert rel < 2e-4, (case, synth.NAMES[wt], no, n_in, seed, rel)
        elif kind == "acc":
            wt, no, rows = rng.choice(FMTS), rng.choice([1, 16, 17, 300, 2048]), rng.randint(1, 8)
            w, x = synth.weights(wt, no, n_in, seed, stream=3), synth.activations(rows, n_in, seed)
            base = synth.activations(rows, no, seed, stream=9)
            y = cuda.gemv(dev(x), dev(w), wt, no, n_in, out=dev(base), accumulate=True).cpu().numpy()
            ok, worst = bound_ok(y, base + g(x, w, wt, no, n_in, rows), oracle.dequant_rows(w, wt, no, n_in), x, 1.1e-4)
            assert ok, (case, synth.NAMES[wt], no, n_in, rows, seed, worst)
        else:
            n_embd, n_ff, n_exp = 256 * rng.randint(1, 8), 256 * rng.randint(1, 6), rng.choice([4, 8, 16])
            k, n_tok = rng.randint(1, min(4, n_exp)), rng.randint(1, 8)
            wg = rng.choice([synth.Q4_K, synth.Q8_0, synth.Q4_0, synth.Q5_K, synth.Q6_K])
            wd = rng.choice([synth.Q6_K, synth.Q4_K, synth.Q8_0, synth.Q4_0, synth.Q5_K])
            gate = [synth.weights(wg, n_ff, n_embd, seed, stream=1000 + e) for e in range(n_exp)]
            up = [synth.weights(wg, n_ff, n_embd, seed, stream=2000 + e) for e in range(n_exp)]
            down = [synth.weights(wd, n_embd, n_ff, seed, stream=3000 + e) for e in range(n_exp)]
            x, logits = synth.activations(n_tok, n_embd, seed), synth.activations(n_tok, n_exp, seed, stream=7)
            ids_ref, wts_ref = oracle.route(logits, k)
            bank = cuda.make_bank(dev(np.stack(gate)), dev(np.stack(up)), dev(np.stack(down)), wg, wd, n_exp, 0, n_embd, n_ff)
            y, ids, _ = cuda.moe_ffn_routed(dev(x), dev(logits), k, bank)
            assert np.array_equal(ids.cpu().numpy(), ids_ref), (case, seed)
            ref = oracle.moe_ffn(x, ids_ref, wts_ref, gate, up, down, wg, wd, n_embd, n_ff, threads=8)
            rel = np.linalg.norm(y.cpu().numpy() - ref) / max(np.linalg.norm(ref), 1e-30)
            assert rel < 2e-4, (case, wg, wd, n_embd, n_ff, n_exp, k, n_tok, seed, rel)
        assert cuda.device_status() == 0
