"""Sharded head and sharded expert bank with two CPU ranks over gloo: the host-side logic of the
multi-GPU path (splits, padding, gather, rank-order sum), with the CPU checker as the compute."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kraken_b200 import shard, synth


def test_row_range_properties():
    for n, world, align in ((128256, 8, 8), (128256, 2, 8), (1001, 4, 8), (7, 4, 1), (5, 8, 1), (0, 2, 8), (16, 3, 16)):
        spans = [shard.row_range(n, world, r, align) for r in range(world)]
        assert sum(c for _, c in spans) == n
        pos = 0
        for b, c in spans:
            assert b == pos or c == 0
            assert b % align == 0 or c == 0
            pos += c
        counts = [c for _, c in spans if c]
        if counts:
            assert max(counts) - min(counts) < 2 * align
    assert shard.row_range(128256, 8, 3, 8) == (3 * 16032, 16032)         # the head of config 4 splits evenly
    assert [shard.expert_range(128, 8, r) for r in (0, 7)] == [(0, 16), (112, 16)]
    with pytest.raises(ValueError):
        shard.row_range(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n_out, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.krk_oracle import Oracle
        orc = Oracle()
        seed = synth.BASE_SEED + 4
        # ---- head: rows split over the ranks, slices generated independently by each rank ----
        n_in = 512
        x = synth.activations(2, n_in, seed)
        probe = shard.ShardedHead(n_out, lambda v: None, align=8)
        w_local = synth.weights(synth.Q6_K, probe.count, n_in, seed, stream=9, row_begin=probe.begin)
        head = shard.ShardedHead(
            n_out, lambda v: torch.from_numpy(orc.gemm(v.numpy(), w_local, synth.Q6_K, probe.count, n_in, rows=v.shape[0])),
            align=8)
        logits = head.forward(torch.from_numpy(x)).numpy()
        w_full = synth.weights(synth.Q6_K, n_out, n_in, seed, stream=9)
        want = orc.gemm(x, w_full, synth.Q6_K, n_out, n_in, rows=2)
        assert logits.shape == want.shape and logits.tobytes() == want.tobytes()    # sharding changes no bit
        # ---- experts: 6 experts over the ranks, top-3, 4 tokens ----
        n_embd, n_ff, n_exp, k, n_tok = 256, 256, 6, 3, 4
        gate = [synth.weights(synth.Q4_K, n_ff, n_embd, seed, stream=100 + e) for e in range(n_exp)]
        up = [synth.weights(synth.Q4_K, n_ff, n_embd, seed, stream=200 + e) for e in range(n_exp)]
        down = [synth.weights(synth.Q6_K, n_embd, n_ff, seed, stream=300 + e) for e in range(n_exp)]
        xm = synth.activations(n_tok, n_embd, seed, stream=5)
        rl = synth.activations(n_tok, n_exp, seed, stream=6)
        base, n_local = shard.expert_range(n_exp, world, rank)
        keep = lambda mats: [m if base <= e < base + n_local else None for e, m in enumerate(mats)]

        def route_fn(lg):
            ids, wts = orc.route(lg.numpy(), k)
            return torch.from_numpy(ids), torch.from_numpy(wts)

        def local_fn(xv, ids, wts):
            return torch.from_numpy(orc.moe_ffn(xv.numpy(), ids.numpy(), wts.numpy(), keep(gate), keep(up), keep(down),
                                                synth.Q4_K, synth.Q6_K, n_embd, n_ff))
        moe = shard.ShardedMoE(n_exp, route_fn, local_fn)
        assert (moe.expert_base, moe.n_local) == (base, n_local)
        y = moe.forward(torch.from_numpy(xm), torch.from_numpy(rl)).numpy()
        ids, wts = orc.route(rl, k)
        assert sum(moe.picks_per_rank(torch.from_numpy(ids))) == n_tok * k
        whole = orc.moe_ffn(xm, ids, wts, gate, up, down, synth.Q4_K, synth.Q6_K, n_embd, n_ff)
        assert np.allclose(y, whole, rtol=1e-5, atol=1e-5 * np.abs(whole).max())
        # every rank holds the same bits (rank-order sum), and they equal the partials added in rank order
        gathered = [torch.empty_like(torch.from_numpy(y)) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(y))
        assert all(torch.equal(g, gathered[0]) for g in gathered)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_out", [96, 101])     # even split, and one that needs padding
def test_two_ranks_over_gloo(n_out):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, n_out, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        for p in procs:
            if p.is_alive():
                p.kill()          # our own child, by handle
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(ret) == {0: "ok", 1: "ok"}
