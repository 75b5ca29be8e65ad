"""Two GPUs of one box: the fused GEMV + all-gather over peer stores, and the NCCL paths, against the
unsharded kernels. Skipped on a single-GPU box (the host logic is covered on CPU over gloo)."""
import os
import socket

import numpy as np
import pytest

from kraken_b200 import synth

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from kraken_b200 import capi, shard
        seed = synth.BASE_SEED + 44
        n_out, n_in, wt = 4008, 4096, synth.Q6_K
        w_full = torch.from_numpy(synth.weights(wt, n_out, n_in, seed)).cuda()
        begin, count = shard.row_range(n_out, world, rank, 8)
        w_local = w_full[begin:begin + count].contiguous()
        for rows, host_counted in ((1, False), (3, False), (2, True)):
            head = shard.PeerHead(n_out, n_in, wt, w_local, rows=rows, host_counted=host_counted)
            nccl_head = shard.ShardedHead(n_out, shard.cuda_head_fn(w_local, wt, count, n_in), align=8)
            for step in range(5):          # several steps: both buffers, increasing epochs
                x = torch.from_numpy(synth.activations(rows, n_in, seed + step)).cuda()
                want = capi.gemv(x, w_full, wt, n_out, n_in)
                got = head.forward(x)
                torch.cuda.synchronize()
                assert capi.device_status() == 0
                assert torch.equal(got, want), f"peer-store head differs at step {step}"
                assert torch.equal(nccl_head.forward(x), want)
            head.close()
            dist.barrier()
        # ---- expert-sharded FFN: partial sums through peer stores == through NCCL, and close to the whole ----
        n_embd, n_ff, n_exp, k = 1024, 512, 8, 4
        mk = lambda wt, r, c, st: [synth.weights(wt, r, c, seed, stream=st + e) for e in range(n_exp)]
        gate, up, down = mk(synth.Q4_K, n_ff, n_embd, 1000), mk(synth.Q4_K, n_ff, n_embd, 2000), mk(synth.Q6_K, n_embd, n_ff, 3000)
        stack = lambda mats, lo, hi: torch.from_numpy(np.stack(mats[lo:hi])).cuda()
        whole = capi.make_bank(stack(gate, 0, n_exp), stack(up, 0, n_exp), stack(down, 0, n_exp), synth.Q4_K, synth.Q6_K,
                               n_exp, 0, n_embd, n_ff)
        base, n_local = shard.expert_range(n_exp, world, rank)
        bank = capi.make_bank(stack(gate, base, base + n_local), stack(up, base, base + n_local),
                              stack(down, base, base + n_local), synth.Q4_K, synth.Q6_K, n_local, base, n_embd, n_ff)
        route_fn, local_fn, combine_fn = shard.cuda_moe_fns(bank, k)
        peer_sum = shard.PeerSum(8 * n_embd)
        moe_peer = shard.ShardedMoE(n_exp, route_fn, local_fn, combine_fn, exchange=peer_sum)
        moe_nccl = shard.ShardedMoE(n_exp, route_fn, local_fn, combine_fn)
        for step, n_tok in enumerate((1, 8, 3, 8, 1)):
            x = torch.from_numpy(synth.activations(n_tok, n_embd, seed + 50 + step)).cuda()
            logits = torch.from_numpy(synth.activations(n_tok, n_exp, seed + 60 + step, stream=7)).cuda()
            got = moe_peer.forward(x, logits).clone()
            via_nccl = moe_nccl.forward(x, logits)
            torch.cuda.synchronize()
            assert capi.device_status() == 0
            assert torch.equal(got, via_nccl), f"peer-store exchange differs from NCCL at step {step}"
            ids, wts = capi.route(logits, k)
            ref = capi.moe_ffn(x, ids, wts, whole)
            rel = float((got - ref).norm() / ref.norm())
            assert rel < 1e-5, rel
        peer_sum.close()
        dist.barrier()
        # ---- the C-side exchange: krk_cuda_shard_allgather over a communicator made by the library's own wrappers ----
        ids = [capi.NcclComm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = capi.NcclComm(world, rank, ids[0])
        even = (n_out // world) // 8 * 8                      # equal slices for the plain all-gather
        x = torch.from_numpy(synth.activations(1, n_in, seed + 90)).cuda()
        mine = capi.gemv(x, w_full[rank * even:(rank + 1) * even].contiguous(), wt, even, n_in)
        full = torch.zeros((world, even), dtype=torch.float32, device="cuda")
        comm.allgather(full, mine)
        torch.cuda.synchronize()
        want = capi.gemv(x, w_full[:world * even].contiguous(), wt, world * even, n_in)
        assert torch.equal(full.view(1, -1), want), "C-side NCCL all-gather of the slices differs from the unsharded row"
        full[rank].copy_(mine[0] * 2)                          # in place: the slice already sits in its slot
        comm.allgather(full, full[rank])
        torch.cuda.synchronize()
        assert torch.equal(full.view(1, -1), want * 2)
        comm.close()
        dist.barrier()
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_two_gpus_peer_head_and_nccl_head():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
        for p in procs:
            if p.is_alive():
                p.kill()          # our own child, by handle
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(ret) == {0: "ok", 1: "ok"}
