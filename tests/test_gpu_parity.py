"""Parity of the CUDA path with the CPU checker, through the C ABI, on a B200.

Bars (from the task's north star): decoded blocks bit-exact; GEMV |y - y_ref| <= 1e-4 *
||w_row|| * ||x||; every integer result (router ids) exact.
"""
import numpy as np
import pytest

from conftest import bound_ok
from kraken_b200 import synth

pytestmark = pytest.mark.gpu

FMTS = [synth.Q8_0, synth.Q4_0, synth.Q4_K, synth.Q6_K]
GEMV_TOL = 1e-4
SEED = synth.BASE_SEED


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_gemv(cuda, oracle, wt, n_out, n_in, rows, seed, random_payload=False, accumulate=False, expect_stream=None):
    before = cuda.family_count(cuda.FAMILY_GEMV_STREAM), cuda.family_count(cuda.FAMILY_GEMV_GENERIC)
    w = synth.weights(wt, n_out, n_in, seed, stream=wt, random_payload=random_payload)
    x = synth.activations(rows, n_in, seed)
    y_ref = oracle.gemm(x, w, wt, n_out, n_in, rows=rows, threads=8)
    if accumulate:
        base = synth.activations(rows, n_out, seed, stream=2000)
        y = cuda.gemv(dev(x), dev(w), wt, n_out, n_in, out=dev(base), accumulate=True).cpu().numpy()
        y_ref = base + y_ref
    else:
        y = cuda.gemv(dev(x), dev(w), wt, n_out, n_in).cpu().numpy()
    w_deq = oracle.dequant_rows(w, wt, n_out, n_in)
    ok, worst = bound_ok(y, y_ref, w_deq, x, GEMV_TOL)
    assert ok, f"wt={wt} {n_out}x{n_in} rows={rows}: worst error is {worst:.3f} of the bound"
    assert cuda.device_status() == 0
    after = cuda.family_count(cuda.FAMILY_GEMV_STREAM), cuda.family_count(cuda.FAMILY_GEMV_GENERIC)
    if expect_stream is True:
        assert after[0] == before[0] + 1 and after[1] == before[1], "the streaming kernel did not take this shape"
    elif expect_stream is False:
        assert after[0] == before[0] and after[1] == before[1] + 1
    return worst


# ---- decode: bit-exact --------------------------------------------------------------------

@pytest.mark.parametrize("wt", FMTS)
@pytest.mark.parametrize("random_payload", [False, True])
def test_dequant_bit_exact(cuda, oracle, wt, random_payload):
    for n_rows, n_in in ((1, 256), (5, 1536), (64, 4096), (3, 11008)):
        w = synth.weights(wt, n_rows, n_in, SEED + 3, stream=wt, random_payload=random_payload)
        got = cuda.dequant_rows(dev(w), wt, n_rows, n_in).cpu().numpy()
        assert got.tobytes() == oracle.dequant_rows(w, wt, n_rows, n_in).tobytes()


def test_dequant_reference_vectors(cuda, golden):
    for wt in FMTS:
        name = synth.NAMES[wt].lower()
        for tag in ("field", "bytes"):
            w = golden[f"{name}_{tag}_w"]
            want = golden[f"{name}_{tag}_deq"]
            got = cuda.dequant_rows(dev(w), wt, want.shape[0], want.shape[1]).cpu().numpy()
            assert got.tobytes() == want.tobytes()
    for key, wt, n in (("kat_q4_0", synth.Q4_0, 32), ("kat_q8_0", synth.Q8_0, 32),
                       ("kat_q4_k", synth.Q4_K, 256), ("kat_q6_k", synth.Q6_K, 256)):
        got = cuda.dequant_rows(dev(golden[f"{key}_w"]), wt, 1, n).cpu().numpy()
        assert got.tobytes() == golden[f"{key}_deq"].tobytes()


def test_dequant_every_scale_bit_pattern(cuda, oracle):
    """All 65536 f16 scale patterns (subnormals, inf, nan included) through one Q8_0 block each."""
    blocks = np.zeros((65536, 34), np.uint8)
    h = np.arange(65536, dtype=np.uint32)
    blocks[:, 0], blocks[:, 1] = h & 0xFF, h >> 8
    blocks[:, 2:] = np.array([1, 255, 127, 129] * 8, np.uint8)
    got = cuda.dequant_rows(dev(blocks), synth.Q8_0, 65536, 32).cpu().numpy()
    want = oracle.dequant_rows(blocks, synth.Q8_0, 65536, 32)
    # A NaN scale gives NaN on both sides; the GPU multiplier returns the canonical NaN while the
    # host keeps the payload, so NaN results are compared as "both NaN", everything else by bits.
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
    assert nan.sum() == 2 * 1023 * 32 and np.isinf(want).sum() == 2 * 32


# ---- GEMV ----------------------------------------------------------------------------------

@pytest.mark.parametrize("wt", FMTS)
@pytest.mark.parametrize("rows", [1, 2, 7, 8])
def test_gemv_shapes(cuda, oracle, wt, rows):
    bs = synth.BLOCK_SIZE[wt]
    for n_out, n_in in ((1, bs), (7, 256), (33, 1536), (257, 4096), (100, 11008), (16, 2048), (300, 512)):
        run_gemv(cuda, oracle, wt, n_out, n_in, rows, SEED + rows)


@pytest.mark.parametrize("wt", FMTS)
def test_gemv_random_bytes_and_accumulate(cuda, oracle, wt):
    run_gemv(cuda, oracle, wt, 129, 2048, 1, SEED + 21, random_payload=True)
    run_gemv(cuda, oracle, wt, 129, 2048, 3, SEED + 22, accumulate=True)
    run_gemv(cuda, oracle, wt, 4096, 4096, 1, SEED + 23, accumulate=True)


def test_gemv_reference_vectors(cuda, golden, oracle):
    for wt in FMTS:
        name = synth.NAMES[wt].lower()
        for tag in ("field", "bytes"):
            w, x, want = golden[f"{name}_{tag}_w"], golden[f"{name}_{tag}_x"], golden[f"{name}_{tag}_y"]
            n_out, n_in = w.shape[0], x.shape[1]
            y = cuda.gemv(dev(x), dev(w), wt, n_out, n_in).cpu().numpy()
            ok, worst = bound_ok(y, want, golden[f"{name}_{tag}_deq"], x, GEMV_TOL)
            assert ok, f"{name}/{tag}: {worst:.3f} of the bound"


def test_config1_q8_0_decode(cuda, oracle):
    """Q8_0 4096x4096, batch 1: the reference's own CPU-runnable case, at full size."""
    run_gemv(cuda, oracle, synth.Q8_0, 4096, 4096, 1, SEED + 1, expect_stream=True)


@pytest.mark.parametrize("shape", [(4096, 4096), (11008, 4096), (4096, 11008)])
def test_config2_q4_k_llama7b_shapes(cuda, oracle, shape):
    run_gemv(cuda, oracle, synth.Q4_K, shape[0], shape[1], 1, SEED + 2, expect_stream=True)


def test_config4_q6_k_head_slice_and_linearity(cuda, oracle):
    """An eighth of the 128256x4096 head against the checker, then the full head through
    size-independent properties: row slices of the full call equal calls on the slices, and
    y(a*x1 + x2) = a*y(x1) + y(x2) within the bound."""
    import torch
    n_in, n_full = 4096, 128256
    run_gemv(cuda, oracle, synth.Q6_K, n_full // 8, n_in, 1, SEED + 4, expect_stream=True)
    part = synth.weights(synth.Q6_K, 2004, n_in, SEED + 4, stream=synth.Q6_K)
    w = dev(part).repeat(64, 1)                                  # 128256 rows, 431 MB
    assert w.shape[0] == n_full
    x1, x2 = synth.activations(1, n_in, SEED + 40), synth.activations(1, n_in, SEED + 41)
    y1 = cuda.gemv(dev(x1), w, synth.Q6_K, n_full, n_in)
    y2 = cuda.gemv(dev(x2), w, synth.Q6_K, n_full, n_in)
    y3 = cuda.gemv(dev(0.5 * x1 + x2), w, synth.Q6_K, n_full, n_in)
    assert torch.equal(y1.view(64, 2004)[0], y1.view(64, 2004)[63])          # repeated rows, same answer
    y_slice = cuda.gemv(dev(x1), w[2004 * 5:], synth.Q6_K, 2004 * 3, n_in)
    assert torch.equal(y_slice.view(-1), y1.view(-1)[2004 * 5:2004 * 8])     # a shard equals its slice
    w_deq = oracle.dequant_rows(part, synth.Q6_K, 2004, n_in)
    ok, worst = bound_ok(y3.cpu().numpy()[:, :2004], (0.5 * y1 + y2).cpu().numpy()[:, :2004], w_deq,
                         np.abs(0.5 * x1) + np.abs(x2), 3 * GEMV_TOL)
    assert ok, worst
    ref = oracle.gemm(x1, part, synth.Q6_K, 2004, n_in, threads=8)
    ok, worst = bound_ok(y1.cpu().numpy()[:, :2004], ref, w_deq, x1, GEMV_TOL)
    assert ok, worst


def test_path_selection(cuda, oracle):
    """Which kernel serves which shape: K not a multiple of 256 takes the
    shape-agnostic kernel; Q6_K rows that are not 16-byte multiples
    (K = 1536) still stream, as whole tiles; every block format streams when K is a multiple of 256 (stacked tiles at K <= 1024)."""
    run_gemv(cuda, oracle, synth.Q4_0, 64, 1024, 1, SEED + 30, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q4_0, 4099, 4096, 1, SEED + 37, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q4_0, 1001, 11008, 1, SEED + 38, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q4_0, 64, 1024, 2, SEED + 39, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q4_0, 333, 4096, 7, SEED + 41, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q5_K, 64, 1024, 1, SEED + 40, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q5_K, 1001, 4096, 1, SEED + 42, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q5_K, 333, 4096, 8, SEED + 43, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q5_K, 77, 11008, 2, SEED + 45, random_payload=True, expect_stream=True)
    for k, wt in enumerate((synth.Q5_0, synth.Q5_1, synth.IQ4_NL, synth.Q2_K, synth.Q3_K)):
        run_gemv(cuda, oracle, wt, 64, 1024, 1, SEED + 44 + 100 * k, expect_stream=True)
        run_gemv(cuda, oracle, wt, 4099, 4096, 1, SEED + 46 + 100 * k, random_payload=True, expect_stream=True)
        run_gemv(cuda, oracle, wt, 1001, 11008, 2, SEED + 47 + 100 * k, random_payload=True, expect_stream=True)
        run_gemv(cuda, oracle, wt, 333, 4096, 3, SEED + 48 + 100 * k, random_payload=True, expect_stream=True)
        run_gemv(cuda, oracle, wt, 77, 2048, 8, SEED + 49 + 100 * k, random_payload=True, expect_stream=True)
        run_gemv(cuda, oracle, wt, 50, 256, 1, SEED + 50 + 100 * k, expect_stream=True)
    # Q2_K / Q3_K rows are 16-byte multiples only for K % 1024 / K % 2048 == 0: both kinds of row, odd unit counts
    for k, wt in enumerate((synth.Q2_K, synth.Q3_K)):
        run_gemv(cuda, oracle, wt, 300, 768, 2, SEED + 51 + 100 * k, random_payload=True, expect_stream=True)
        run_gemv(cuda, oracle, wt, 129, 5120, 1, SEED + 52 + 100 * k, random_payload=True, expect_stream=True)
        run_gemv(cuda, oracle, wt, 64, 8192, 4, SEED + 53 + 100 * k, expect_stream=True)
        run_gemv(cuda, oracle, wt, 40, 1280, 1, SEED + 54 + 100 * k, accumulate=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q8_0, 64, 96, 1, SEED + 31, expect_stream=False)
    run_gemv(cuda, oracle, synth.Q6_K, 4096, 1536, 1, SEED + 32, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 1001, 1536, 8, SEED + 33, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q4_K, 1536, 4096, 8, SEED + 34, expect_stream=True)
    # Q6_K rows that are neither 16-byte multiples nor short enough for whole tiles: copied row by row from the
    # 16-byte boundary below (K = 11008: 9030-byte rows, 2-byte aligned; K = 5120: 4200 bytes; K = 768: stacked tiles)
    run_gemv(cuda, oracle, synth.Q6_K, 4099, 11008, 1, SEED + 60, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 333, 11008, 2, SEED + 61, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 77, 11008, 4, SEED + 62, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 77, 5120, 8, SEED + 69, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 1001, 5120, 1, SEED + 63, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 100, 5120, 4, SEED + 64, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 257, 768, 1, SEED + 65, random_payload=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 40, 768, 3, SEED + 66, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 5, 13824, 1, SEED + 67, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q6_K, 64, 11008, 1, SEED + 68, accumulate=True, expect_stream=True)
    run_gemv(cuda, oracle, synth.Q8_0, 5, 256, 3, SEED + 35, expect_stream=True)


def test_gemv_nonfinite_activation_gives_nan(cuda):
    import torch
    w = dev(synth.weights(synth.Q4_K, 32, 512, SEED + 36))
    x = torch.ones(512, device="cuda")
    x[100] = float("inf")
    assert torch.isnan(cuda.gemv(x, w, synth.Q4_K, 32, 512)).all()
    x[100] = 0.0
    assert torch.isfinite(cuda.gemv(x, w, synth.Q4_K, 32, 512)).all()
    assert (cuda.gemv(torch.zeros(512, device="cuda"), w, synth.Q4_K, 32, 512) == 0).all()
    w0 = dev(synth.weights(synth.Q4_0, 32, 512, SEED + 36))
    x[100] = float("nan")
    assert torch.isnan(cuda.gemv(x, w0, synth.Q4_0, 32, 512)).all()
    x[100] = 0.0
    assert torch.isfinite(cuda.gemv(x, w0, synth.Q4_0, 32, 512)).all()
    for wt in (synth.Q5_0, synth.Q5_1, synth.IQ4_NL, synth.Q2_K, synth.Q3_K, synth.Q5_K, synth.Q6_K, synth.Q8_0):
        w5 = dev(synth.weights(wt, 32, 512, SEED + 36))
        x[77] = float("-inf")
        assert torch.isnan(cuda.gemv(x, w5, wt, 32, 512)).all()
        x[77] = 0.0
        assert torch.isfinite(cuda.gemv(x, w5, wt, 32, 512)).all()


def test_gemv_empty_and_refusals(cuda):
    import torch
    x = torch.zeros(256, device="cuda")
    w = torch.zeros(144 * 4, dtype=torch.uint8, device="cuda")
    assert cuda.gemv(x, w, synth.Q4_K, 0, 256).shape == (1, 0)
    before = cuda.launch_count()
    with pytest.raises(cuda.KrkCudaError) as e:
        cuda.gemv(x[:100], w, synth.Q4_K, 4, 100)
    assert e.value.rc == -2
    with pytest.raises(cuda.KrkCudaError) as e:
        cuda.gemv(x, w, 99, 4, 256)
    assert e.value.rc == -1
    with pytest.raises(cuda.KrkCudaError) as e:
        cuda.gemv(x, w[8:], synth.Q4_K, 3, 256)
    assert e.value.rc == -4
    assert cuda.launch_count() == before


# ---- grouped GEMV ----------------------------------------------------------------------------

def test_gemv_group_shared_x_and_silu_pair(cuda, oracle):
    n_in, n_ff = 4096, 1536
    seed = SEED + 6
    x = synth.activations(1, n_in, seed)
    ws = [synth.weights(synth.Q4_K, n, n_in, seed, stream=100 + i) for i, n in enumerate((n_ff, n_ff, 512, 40))]
    n_outs = [w.shape[0] for w in ws]
    dx = dev(x)
    outs = cuda.gemv_group([dx] * 4, [dev(w) for w in ws], [synth.Q4_K] * 4, n_outs, n_in)
    for w, y in zip(ws, outs):
        ref = oracle.gemm(x, w, synth.Q4_K, w.shape[0], n_in)
        ok, worst = bound_ok(y.cpu().numpy()[None], ref, oracle.dequant_rows(w, synth.Q4_K, w.shape[0], n_in), x, GEMV_TOL)
        assert ok, worst
    # the gate/up fold: y[0] = silu(gate) * up
    outs = cuda.gemv_group([dx] * 2, [dev(ws[0]), dev(ws[1])], [synth.Q4_K] * 2, n_outs[:2], n_in, fuse_silu_pair=True)
    g = oracle.gemm(x, ws[0], synth.Q4_K, n_ff, n_in)
    u = oracle.gemm(x, ws[1], synth.Q4_K, n_ff, n_in)
    want = oracle.silu_mul(g, u)[0]
    got = outs[0].cpu().numpy()
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-4 * scale + 1e-6


def test_gemv_group_own_x_mixed_types(cuda, oracle):
    n_in = 1536
    seed = SEED + 7
    wts = [synth.Q6_K, synth.Q6_K, synth.Q8_0, synth.Q4_0]
    n_outs = [4096, 300, 64, 33]
    ws = [synth.weights(wt, n, n_in, seed, stream=200 + i) for i, (wt, n) in enumerate(zip(wts, n_outs))]
    xs = [synth.activations(1, n_in, seed, stream=300 + i) for i in range(4)]
    outs = cuda.gemv_group([dev(x) for x in xs], [dev(w) for w in ws], wts, n_outs, n_in)
    for wt, w, x, y in zip(wts, ws, xs, outs):
        ref = oracle.gemm(x, w, wt, w.shape[0], n_in)
        ok, worst = bound_ok(y.cpu().numpy()[None], ref, oracle.dequant_rows(w, wt, w.shape[0], n_in), x, GEMV_TOL)
        assert ok, (wt, worst)


def test_gemv_group_ragged_q6k_rows(cuda, oracle):
    """Groups and the gate/up fold over Q6_K rows that are copied from the 16-byte boundary below each row
    (K = 5120 and K = 11008): matrices of one launch start at different offsets into their slots."""
    seed = SEED + 70
    for n_in, n_outs in ((5120, (333, 333, 48)), (11008, (100, 100, 17))):
        x = synth.activations(1, n_in, seed)
        ws = [synth.weights(synth.Q6_K, n, n_in, seed, stream=400 + i, random_payload=(i == 2)) for i, n in enumerate(n_outs)]
        dx = dev(x)
        before = cuda.family_count(cuda.FAMILY_GEMV_STREAM)
        outs = cuda.gemv_group([dx] * 3, [dev(w) for w in ws], [synth.Q6_K] * 3, list(n_outs), n_in)
        assert cuda.family_count(cuda.FAMILY_GEMV_STREAM) == before + 1
        for w, y in zip(ws, outs):
            ref = oracle.gemm(x, w, synth.Q6_K, w.shape[0], n_in)
            ok, worst = bound_ok(y.cpu().numpy()[None], ref, oracle.dequant_rows(w, synth.Q6_K, w.shape[0], n_in), x, GEMV_TOL)
            assert ok, (n_in, worst)
        outs = cuda.gemv_group([dx] * 2, [dev(ws[0]), dev(ws[1])], [synth.Q6_K] * 2, list(n_outs[:2]), n_in, fuse_silu_pair=True)
        g = oracle.gemm(x, ws[0], synth.Q6_K, n_outs[0], n_in)
        u = oracle.gemm(x, ws[1], synth.Q6_K, n_outs[1], n_in)
        want = oracle.silu_mul(g, u)[0]
        got = outs[0].cpu().numpy()
        assert np.abs(got - want).max() <= 2e-4 * np.abs(want).max() + 1e-6
        assert cuda.device_status() == 0


# ---- MoE --------------------------------------------------------------------------------------

def test_route_ids_exact(cuda, oracle):
    import torch
    logits = synth.activations(64, 128, SEED + 8, stream=7)
    logits[3, 10] = logits[3, 99] = logits[3].max() + 1.0        # an exact tie: the lower id wins
    logits[4, :] = 0.25                                           # everything ties
    ids, wts = cuda.route(dev(logits), 8)
    ids_ref, wts_ref = oracle.route(logits, 8)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    assert ids_ref[3, 0] == 10 and ids_ref[3, 1] == 99 and ids_ref[4].tolist() == list(range(8))
    assert np.allclose(wts.cpu().numpy(), wts_ref, rtol=2e-6, atol=1e-9)


def moe_case(cuda, oracle, n_embd, n_ff, n_exp, k, n_tok, seed, local=None, wt_gu=synth.Q4_K, wt_dn=synth.Q6_K):
    import torch
    gate = [synth.weights(wt_gu, n_ff, n_embd, seed, stream=1000 + e) for e in range(n_exp)]
    up = [synth.weights(wt_gu, n_ff, n_embd, seed, stream=2000 + e) for e in range(n_exp)]
    down = [synth.weights(wt_dn, n_embd, n_ff, seed, stream=3000 + e) for e in range(n_exp)]
    x = synth.activations(n_tok, n_embd, seed)
    logits = synth.activations(n_tok, n_exp, seed, stream=7)
    ids_ref, wts_ref = oracle.route(logits, k)
    ids, wts = cuda.route(dev(logits), k)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    lo, hi = local if local else (0, n_exp)
    sel = lambda mats: [m if lo <= e < hi else None for e, m in enumerate(mats)]
    y_ref = oracle.moe_ffn(x, ids_ref, wts_ref, sel(gate), sel(up), sel(down), wt_gu, wt_dn, n_embd, n_ff,
                           threads=8)
    bank = cuda.make_bank(dev(np.stack(gate[lo:hi])), dev(np.stack(up[lo:hi])), dev(np.stack(down[lo:hi])),
                          wt_gu, wt_dn, hi - lo, lo, n_embd, n_ff)
    keep = (bank,)
    y = cuda.moe_ffn(dev(x), ids, wts, bank).cpu().numpy()
    assert cuda.device_status() == 0
    rel = np.linalg.norm(y - y_ref) / max(np.linalg.norm(y_ref), 1e-30)
    assert rel < 2e-4, f"relative L2 error {rel:.2e}"
    return y, y_ref, keep


def test_moe_routed_equals_route_then_ffn(cuda):
    """krk_cuda_moe_ffn_routed gives the bits of krk_cuda_route followed by krk_cuda_moe_ffn, on the streaming
    path (routing folded into the plan kernel) and on the shape-agnostic one, whole bank and a shard."""
    import torch
    for n_embd, n_ff, n_exp, k, n_tok, local in ((4096, 1536, 16, 8, 8, None), (4096, 1536, 16, 8, 1, (8, 16)),
                                                  (512, 768, 8, 2, 3, None)):
        seed = SEED + 70 + n_tok
        lo, hi = local if local else (0, n_exp)
        mk = lambda wt, r, c, st: dev(np.stack([synth.weights(wt, r, c, seed, stream=st + e) for e in range(lo, hi)]))
        bank = cuda.make_bank(mk(synth.Q4_K, n_ff, n_embd, 1000), mk(synth.Q4_K, n_ff, n_embd, 2000),
                              mk(synth.Q6_K, n_embd, n_ff, 3000), synth.Q4_K, synth.Q6_K, hi - lo, lo, n_embd, n_ff)
        x = dev(synth.activations(n_tok, n_embd, seed))
        logits = dev(synth.activations(n_tok, n_exp, seed, stream=7))
        ids, wts = cuda.route(logits, k)
        want = cuda.moe_ffn(x, ids, wts, bank)
        got, ids2, wts2 = cuda.moe_ffn_routed(x, logits, k, bank)
        assert cuda.device_status() == 0
        assert torch.equal(ids, ids2) and torch.equal(wts, wts2)
        assert torch.equal(got, want)


@pytest.mark.parametrize("wt_gu,wt_dn", [(synth.Q4_0, synth.Q8_0), (synth.Q5_K, synth.Q4_K), (synth.Q8_0, synth.Q5_K),
                                          (synth.Q6_K, synth.Q4_0), (synth.Q5_0, synth.Q5_1), (synth.Q5_1, synth.IQ4_NL),
                                          (synth.IQ4_NL, synth.Q2_K), (synth.Q2_K, synth.Q3_K), (synth.Q3_K, synth.Q6_K)])
def test_moe_other_expert_formats(cuda, oracle, wt_gu, wt_dn):
    """Expert banks in the other formats: the device-table launches of every streaming arm, whole bank and a shard.
    Hidden 2048 gives Q6_K / Q3_K rows of 16-byte multiples, expert width 1024 gives Q2_K such rows; the second
    shape (hidden 1280, width 768) makes the rows of all three ragged."""
    moe_case(cuda, oracle, 2048, 1024, 8, 2, 3, SEED + 13, wt_gu=wt_gu, wt_dn=wt_dn)
    moe_case(cuda, oracle, 2048, 1024, 8, 4, 1, SEED + 14, local=(4, 8), wt_gu=wt_gu, wt_dn=wt_dn)
    if wt_gu in (synth.Q6_K, synth.Q2_K, synth.Q3_K) or wt_dn in (synth.Q6_K, synth.Q2_K, synth.Q3_K):
        moe_case(cuda, oracle, 1280, 768, 8, 2, 2, SEED + 15, wt_gu=wt_gu, wt_dn=wt_dn)


def test_moe_small(cuda, oracle):
    moe_case(cuda, oracle, 512, 768, 8, 2, 3, SEED + 9)
    moe_case(cuda, oracle, 256, 512, 4, 4, 1, SEED + 10)        # every expert picked


def test_moe_config5_shapes_and_shards(cuda, oracle):
    """Qwen3-MoE expert shapes (hidden 4096, expert width 1536, top-8) over a 16-expert bank,
    batch 1 and 8; then two 8-expert shards whose partial sums add up to the whole."""
    y1, y1_ref, _ = moe_case(cuda, oracle, 4096, 1536, 16, 8, 1, SEED + 11)
    y8, y8_ref, _ = moe_case(cuda, oracle, 4096, 1536, 16, 8, 8, SEED + 12)
    a, a_ref, _ = moe_case(cuda, oracle, 4096, 1536, 16, 8, 8, SEED + 12, local=(0, 8))
    b, b_ref, _ = moe_case(cuda, oracle, 4096, 1536, 16, 8, 8, SEED + 12, local=(8, 16))
    parts = dev(np.stack([a, b]))
    total = cuda.sum_parts(parts).cpu().numpy()
    assert np.array_equal(total, a + b)
    assert np.linalg.norm(total - y8_ref) / np.linalg.norm(y8_ref) < 2e-4


def test_silu_mul_and_scatter(cuda, golden):
    got = cuda.silu_mul(dev(golden["silu_gate"]), dev(golden["silu_up"])).cpu().numpy()
    assert np.allclose(got, golden["silu_out"], rtol=3e-6, atol=1e-7)
    dst = dev(golden["scatter_dst"])
    cuda.scatter_axpy_rows(dst, dev(golden["scatter_src"]), dev(golden["scatter_rows"]), dev(golden["scatter_alpha"]))
    assert dst.cpu().numpy().tobytes() == golden["scatter_out"].tobytes()


def test_gather_rows_then_scatter_is_the_weighted_permute(cuda, oracle):
    """gather_rows (include/krk/backend.hpp:1451) against the oracle's row move, bit for bit, on aligned and odd
    row lengths, repeated and empty index lists; then gather -> scatter_axpy_rows with alpha 1 onto zeros puts
    every picked row back where it came from."""
    import torch
    rng = np.random.default_rng(SEED + 70)
    for n_src, n, n_rows in ((64, 4096, 23), (9, 1537, 9), (5, 8, 0), (300, 1536, 300)):
        src = rng.standard_normal((n_src, n)).astype(np.float32)
        rows = rng.integers(0, n_src, n_rows).astype(np.int32)
        dst = torch.empty((n_rows, n), dtype=torch.float32, device="cuda")
        cuda.gather_rows(dst, dev(src), dev(rows))
        assert dst.cpu().numpy().tobytes() == oracle.gather_rows(src, rows).tobytes()
    src = rng.standard_normal((40, 1536)).astype(np.float32)
    rows = rng.permutation(40)[:17].astype(np.int32)
    picked = torch.empty((17, 1536), dtype=torch.float32, device="cuda")
    cuda.gather_rows(picked, dev(src), dev(rows))
    back = torch.zeros((40, 1536), dtype=torch.float32, device="cuda")
    cuda.scatter_axpy_rows(back, picked, dev(rows), dev(np.ones(17, np.float32)))
    want = np.zeros_like(src)
    want[rows] = src[rows]
    assert back.cpu().numpy().tobytes() == want.tobytes()


# ---- the host-buffer boundary: CudaBackend -------------------------------------------------------

def test_backend_host_buffers_roundtrip(cuda, oracle):
    """upload -> gemm / gemm_accumulate / gemm_group -> download with host arrays, as a Kraken
    engine drives a backend (include/krk/backend.hpp:720-770, 858-900, 1040-1056)."""
    be = cuda.Backend(0)
    assert "sm_100" in be.describe()
    n_out, n_in = 1000, 4096
    wt = synth.Q4_K
    w = synth.weights(wt, n_out, n_in, SEED + 13)
    x = synth.activations(2, n_in, SEED + 13)
    assert be.gemm_k_ok(wt, n_in) and not be.gemm_k_ok(wt, 100)
    d_w, d_x, d_y = be.alloc(w.nbytes), be.alloc(x.nbytes), be.alloc(2 * n_out * 4)
    be.upload(d_w, w.ctypes.data, w.nbytes)
    be.upload(d_x, x.ctypes.data, x.nbytes)
    be.gemm(d_y, d_x, d_w, wt, n_out, n_in, 2)
    y = np.empty((2, n_out), np.float32)
    be.download(y.ctypes.data, d_y, y.nbytes)
    ref = oracle.gemm(x, w, wt, n_out, n_in, rows=2, threads=8)
    w_deq = oracle.dequant_rows(w, wt, n_out, n_in)
    ok, worst = bound_ok(y, ref, w_deq, x, GEMV_TOL)
    assert ok, worst
    assert be.gemm_accumulate(d_y, d_x, d_w, wt, n_out, n_in, 2)
    y2 = np.empty_like(y)
    be.download(y2.ctypes.data, d_y, y2.nbytes)
    ok, worst = bound_ok(y2, 2 * ref, w_deq, 2 * x, GEMV_TOL)
    assert ok, worst
    d_y2 = be.alloc(n_out * 4)
    be.fill0(d_y2, n_out * 4)
    ran, fused = be.gemm_group([d_y, d_y2], d_x, [d_w, d_w], wt, [n_out, n_out], n_in, rows=1, silu=True)
    assert ran and fused
    h = np.empty(n_out, np.float32)
    be.download(h.ctypes.data, d_y, h.nbytes)
    want = oracle.silu_mul(ref[0], ref[0])
    assert np.abs(h - want).max() <= 2e-4 * np.abs(want).max()
    for p in (d_w, d_x, d_y, d_y2):
        be.release(p)
    be.close()


def test_decode_layer_matmuls_through_backend(cuda, oracle):
    """The matmuls of one decode layer as Kraken's engine issues them on a backend (include/krk/backend.hpp:
    858-900, 1040-1056): q/k/v in one gemm_group, the attention output folded into the residual with
    gemm_accumulate, gate/up in one gemm_group with the silu fold, the down projection folded into the
    residual. Mixed formats as in a Q4_K_M file (Q4_K projections, Q6_K value and down). Attention itself is
    out of scope: q stands in for its output. Checked against the oracle's composition of the same steps."""
    be = cuda.Backend(0)
    n_embd, n_ff, n_kv = 1024, 2816, 256
    seed = SEED + 21
    mk = lambda wt, n, k, st: synth.weights(wt, n, k, seed, stream=st)
    wq, wk = mk(synth.Q4_K, n_embd, n_embd, 1), mk(synth.Q4_K, n_kv, n_embd, 2)
    wv, wo = mk(synth.Q6_K, n_kv, n_embd, 3), mk(synth.Q4_K, n_embd, n_embd, 4)
    wg, wu = mk(synth.Q4_K, n_ff, n_embd, 5), mk(synth.Q4_K, n_ff, n_embd, 6)
    wd = mk(synth.Q6_K, n_embd, n_ff, 7)
    x = synth.activations(1, n_embd, seed)
    resid0 = synth.activations(1, n_embd, seed, stream=9)

    def up(a):
        p = be.alloc(a.nbytes)
        be.upload(p, a.ctypes.data, a.nbytes)
        return p

    def down(p, n):
        out = np.empty(n, np.float32)
        be.download(out.ctypes.data, p, out.nbytes)
        return out

    d = {k: up(v) for k, v in dict(wq=wq, wk=wk, wv=wv, wo=wo, wg=wg, wu=wu, wd=wd, x=x, resid=resid0).items()}
    d_q, d_k, d_v, d_h, d_u = (be.alloc(4 * n) for n in (n_embd, n_kv, n_kv, n_ff, n_ff))
    # q, k (same type) in one group; v has another type, so it goes alone, as Backend::gemm_group's `wt` asks
    ran, _ = be.gemm_group([d_q, d_k], d["x"], [d["wq"], d["wk"]], synth.Q4_K, [n_embd, n_kv], n_embd, rows=1)
    assert ran
    be.gemm(d_v, d["x"], d["wv"], synth.Q6_K, n_kv, n_embd, 1)
    assert be.gemm_accumulate(d["resid"], d_q, d["wo"], synth.Q4_K, n_embd, n_embd, 1)       # resid += Wo . attn
    ran, fused = be.gemm_group([d_h, d_u], d["resid"], [d["wg"], d["wu"]], synth.Q4_K, [n_ff, n_ff], n_embd, rows=1, silu=True)
    assert ran and fused                                                                   # h = silu(Wg r) * (Wu r)
    assert be.gemm_accumulate(d["resid"], d_h, d["wd"], synth.Q6_K, n_embd, n_ff, 1)          # resid += Wd . h

    g = lambda xx, w, wt, n, k: oracle.gemm(xx, w, wt, n, k, rows=1, threads=8)
    q_ref, k_ref, v_ref = g(x, wq, synth.Q4_K, n_embd, n_embd), g(x, wk, synth.Q4_K, n_kv, n_embd), g(x, wv, synth.Q6_K, n_kv, n_embd)
    r1 = resid0 + g(q_ref, wo, synth.Q4_K, n_embd, n_embd)
    h_ref = oracle.silu_mul(g(r1, wg, synth.Q4_K, n_ff, n_embd)[0], g(r1, wu, synth.Q4_K, n_ff, n_embd)[0])[None, :]
    r2 = r1 + g(h_ref, wd, synth.Q6_K, n_embd, n_ff)
    for name, got, want in (("q", down(d_q, n_embd), q_ref[0]), ("k", down(d_k, n_kv), k_ref[0]), ("v", down(d_v, n_kv), v_ref[0]),
                            ("h", down(d_h, n_ff), h_ref[0]), ("resid", down(d["resid"], n_embd), r2[0])):
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert rel < 2e-5, f"{name}: relative L2 error {rel:.2e}"
    assert cuda.device_status() == 0
    for p in list(d.values()) + [d_q, d_k, d_v, d_h, d_u]:
        be.release(p)
    be.close()


def test_backend_gemm_group_with_per_matrix_types_and_activations(cuda, oracle):
    """Backend::gemm_group's optional arrays (include/krk/backend.hpp:1040-1056): `wts` (q/k/v of a mixed file in
    ONE group: Q4_K, Q4_K, Q6_K) and `xs` (the routed experts' down projections, each reading its own row)."""
    be = cuda.Backend(0)
    n_in, seed = 1024, SEED + 50
    shapes = [(512, synth.Q4_K), (256, synth.Q4_K), (256, synth.Q6_K), (128, synth.Q8_0)]
    ws = [synth.weights(wt, n, n_in, seed, stream=10 + i) for i, (n, wt) in enumerate(shapes)]
    xs = [synth.activations(1, n_in, seed, stream=20 + i) for i in range(len(shapes))]

    def up(a):
        p = be.alloc(a.nbytes)
        be.upload(p, a.ctypes.data, a.nbytes)
        return p

    d_w, d_x = [up(w) for w in ws], [up(x) for x in xs]
    d_y = [be.alloc(4 * n) for n, _ in shapes]
    for use_xs in (False, True):
        ran, fused = be.gemm_group(d_y, d_x[0], d_w, synth.Q4_K, [n for n, _ in shapes], n_in, rows=1,
                                   wts=[wt for _, wt in shapes], xs=d_x if use_xs else None)
        assert ran and not fused
        for i, (n, wt) in enumerate(shapes):
            got = np.empty(n, np.float32)
            be.download(got.ctypes.data, d_y[i], got.nbytes)
            x = xs[i] if use_xs else xs[0]
            ref = oracle.gemm(x, ws[i], wt, n, n_in, rows=1, threads=4)
            ok, worst = bound_ok(got[None, :], ref, oracle.dequant_rows(ws[i], wt, n, n_in), x, GEMV_TOL)
            assert ok, (i, use_xs, worst)
    assert cuda.device_status() == 0
    for p in d_w + d_x + d_y:
        be.release(p)
    be.close()


@pytest.mark.parametrize("wt,n_in", [(synth.Q8_0, 96), (synth.Q8_0, 4128), (synth.Q4_0, 160), (synth.Q5_0, 96)])
@pytest.mark.parametrize("rows", [9, 40])
def test_backend_gemm_fallback_rung_k_not_multiple_of_256(cuda, oracle, wt, n_in, rows):
    """More than eight activation rows with a K that is whole 32-value blocks but not a multiple of 256 (legal
    for the 32-value formats): Backend::gemm_k_ok says yes (include/krk/backend.hpp:862-869), so gemm() must
    compute it (the place of the reference's fallback GEMM, src/hip/kernels/gemm.hpp:1013-1134), not abort."""
    be = cuda.Backend(0)
    n_out = 77
    assert be.gemm_k_ok(wt, n_in)
    w = synth.weights(wt, n_out, n_in, SEED + 21, stream=wt)
    x = synth.activations(rows, n_in, SEED + 21)
    d_w, d_x, d_y = be.alloc(w.nbytes), be.alloc(x.nbytes), be.alloc(rows * n_out * 4)
    be.upload(d_w, w.ctypes.data, w.nbytes)
    be.upload(d_x, x.ctypes.data, x.nbytes)
    be.gemm(d_y, d_x, d_w, wt, n_out, n_in, rows)
    y = np.empty((rows, n_out), np.float32)
    be.download(y.ctypes.data, d_y, y.nbytes)
    ref = oracle.gemm(x, w, wt, n_out, n_in, rows=rows, threads=4)
    ok, worst = bound_ok(y, ref, oracle.dequant_rows(w, wt, n_out, n_in), x, GEMV_TOL)
    assert ok, worst
    for p in (d_w, d_x, d_y):
        be.release(p)
    be.close()
