"""Sharding of the output head and of the routed-expert bank over the GPUs of one box.

The reference has no multi-GPU path at all (one process, one device, one stream:
src/hip/backend_hip.hip:5036-5043), so nothing here replaces a reference file; the two
shardings follow from the shape of the matmul itself:

* output rows are independent dot products (the reference's CPU pool splits them the same way,
  src/backend_cpu.cpp:1274-1276), so GPU g owns a contiguous block of rows of the head, computes
  its slice of the logits, and one all-gather over NVLink assembles the row on every rank;
* experts are independent until the weighted sum, so expert e lives on GPU e // (n_expert/G),
  every rank runs the same deterministic routing on the replicated logits, computes the partial
  sum of the picks it holds, and the partials are all-gathered and added in rank order (rank
  order = ascending expert id blocks, so the result does not depend on timing).

One process per GPU; ``torch.distributed`` carries the collectives (NCCL on GPUs, gloo in the CPU
tests). The compute is injected as a callable so that the same logic runs over the CUDA library
(``cuda_head_fn`` / ``cuda_moe_fn``) or, in the tests, over the CPU checker.
"""
from __future__ import annotations

from typing import Callable, Tuple


def row_range(n: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Contiguous, balanced split of ``n`` rows in units of ``align``: (begin, count) of ``rank``.

    The first ``units % world`` ranks take one more unit; a tail shorter than ``align`` goes to
    the last non-empty rank. Counts sum to ``n`` and begins are multiples of ``align``.
    """
    if world <= 0 or not 0 <= rank < world or n < 0 or align <= 0:
        raise ValueError("bad split arguments")
    units = (n + align - 1) // align
    q, r = divmod(units, world)
    first = rank * q + min(rank, r)
    count = q + (1 if rank < r else 0)
    begin = min(first * align, n)
    end = min((first + count) * align, n)
    return begin, end - begin


def expert_range(n_expert: int, world: int, rank: int) -> Tuple[int, int]:
    """(expert_base, n_local): contiguous blocks, ascending with the rank."""
    return row_range(n_expert, world, rank, 1)


class ShardedHead:
    """logits[rows, n_out] = x . W^T with the rows of W split over the ranks of ``group``.

    ``local_fn(x) -> [rows, count]`` computes this rank's slice (f32). ``forward`` returns the
    full row on every rank. Slices of unequal length are padded to the longest for the
    collective and trimmed afterwards.
    """

    def __init__(self, n_out: int, local_fn: Callable, group=None, align: int = 8):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_out = n_out
        self.ranges = [row_range(n_out, self.world, r, align) for r in range(self.world)]
        self.begin, self.count = self.ranges[self.rank]
        self.max_count = max(c for _, c in self.ranges)
        self.even = all(c == self.max_count for _, c in self.ranges)
        self.local_fn = local_fn
        self._gather = None

    def forward(self, x):
        import torch
        local = self.local_fn(x)                                   # [rows, count]
        rows = local.shape[0]
        if self.world == 1:
            return local
        if self._gather is None or self._gather.shape[1] != rows or self._gather.device != local.device:
            # the collective concatenates along dim 0: [world * rows, max_count], viewed per rank below
            self._flat = torch.empty((self.world * rows, self.max_count), dtype=local.dtype, device=local.device)
            self._gather = self._flat.view(self.world, rows, self.max_count)
            self._pad = torch.zeros((rows, self.max_count), dtype=local.dtype, device=local.device)
        if self.even:
            send = local.contiguous()
        else:
            self._pad[:, :self.count] = local
            send = self._pad
        self.dist.all_gather_into_tensor(self._flat, send, group=self.group)
        if self.even:
            return self._gather.permute(1, 0, 2).reshape(rows, self.n_out)
        return torch.cat([self._gather[r, :, :c] for r, (_, c) in enumerate(self.ranges)], dim=1)


class NcclHead:
    """The NCCL form of the sharded head through the C ABI (krk_cuda_shard_allgather over ncclAllGather): the GEMV
    writes this rank's slice straight into its slot of a persistent full-row buffer and the all-gather runs in
    place on it, so a step is one kernel and one collective with no staging copy; both replay from a CUDA
    graph. Needs slices of equal length (n_out a multiple of world * align) and one activation row. The
    communicator is the library's own (krk_cuda_nccl_comm_init); its id travels through the process group."""

    def __init__(self, n_out: int, n_in: int, wt: int, w_local, group=None, align: int = 8):
        import torch
        import torch.distributed as dist
        from . import capi
        self.capi = capi
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.begin, self.count = row_range(n_out, self.world, self.rank, align)
        if self.count * self.world != n_out:
            raise ValueError("NcclHead needs equal slices")
        self.n_out, self.n_in, self.wt, self.w_local = n_out, n_in, wt, w_local
        ids = [capi.NcclComm.unique_id() if self.rank == 0 else None]
        dist.broadcast_object_list(ids, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self.comm = capi.NcclComm(self.world, self.rank, ids[0])
        self.full = torch.zeros((1, n_out), dtype=torch.float32, device=w_local.device)
        self.slot = self.full[:, self.begin:self.begin + self.count]

    def forward(self, x):
        slot = self.full.view(-1)[self.begin:self.begin + self.count]
        self.capi.gemv(x, self.w_local, self.wt, self.count, self.n_in, out=slot.view(1, -1))
        self.comm.allgather(self.full, slot)
        return self.full

    def gather_only(self):
        slot = self.full.view(-1)[self.begin:self.begin + self.count]
        self.comm.allgather(self.full, slot)
        return self.full

    def close(self):
        self.comm.close()


class _PeerBuffers:
    """A set of device buffers per GPU that every process of the group has mapped: ``own[i]`` is this
    GPU's i-th buffer (capi.PeerBuffer), ``ptrs[i][q]`` its address on GPU q as seen from this process.
    The 64-byte handles travel through the process group."""

    def __init__(self, capi, sizes, group=None):
        import torch.distributed as dist
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.own = [capi.PeerBuffer.alloc(n) for n in sizes]
        everyone = [None] * self.world
        dist.all_gather_object(everyone, [buf.handle for buf in self.own], group=group)
        self.mapped = []
        self.ptrs = [[] for _ in sizes]
        for q, handles in enumerate(everyone):
            if q == self.rank:
                bufs = self.own
            else:
                bufs = [capi.PeerBuffer.open(h, n) for h, n in zip(handles, sizes)]
                self.mapped.append(bufs)
            for i, buf in enumerate(bufs):
                self.ptrs[i].append(buf.ptr)
        dist.barrier(group=group)

    def close(self):
        """Unmap the peers' buffers, then (after a barrier: nobody still maps ours) free our own."""
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        for bufs in self.mapped:
            for buf in bufs:
                buf.release()
        self.mapped = []
        dist.barrier(group=self.group)
        for buf in self.own:
            buf.release()
        self.own = []


class PeerSum:
    """combine step of ShardedMoE over NVLink peer stores (krk_cuda_allgather_sum): ``PeerSum(n_max)(part)``
    returns ((p0 + p1) + p2) + ... over the ranks' partial sums, the same bits on every GPU, from one kernel
    that stores this GPU's part into every GPU's gather buffer, waits (bounded) for the peers and adds."""

    def __init__(self, n_max: int, group=None):
        import torch.distributed as dist
        from . import capi
        self.capi = capi
        world = dist.get_world_size(group)
        self.slot = (n_max + 3) // 4 * 4
        self.bufs = _PeerBuffers(capi, [2 * world * self.slot * 4, 4 * (world + 2)], group)
        self.rank = self.bufs.rank
        self._out = None

    def __call__(self, part):
        import torch
        if part.numel() > self.slot or part.numel() % 4:
            raise ValueError("partial sum larger than the gather slot, or not a multiple of 4 floats")
        if self._out is None or self._out.shape != part.shape:
            self._out = torch.empty_like(part)
        return self.capi.allgather_sum(self.bufs.ptrs[0], self.bufs.ptrs[1], self.rank, self.slot, part.contiguous(), self._out)

    def close(self):
        self.bufs.close()


class PeerHead:
    """Row-sharded head whose GEMV epilogue stores its slice straight into every GPU's copy of the logits
    row (krk_cuda_gemv_allgather): compute and all-gather are one kernel over NVLink peer memory, whose last
    CTA waits (bounded) for the peers' slices; ``host_counted`` keeps the wait as a second small kernel. Two output buffers alternate so that a fast rank's next step never overwrites a
    row a slow rank still reads. One process per GPU of one box; the buffers come from krk_cuda_peer_alloc and
    their 64-byte handles travel through the process group. Results are bit-identical to the unsharded GEMV.
    """

    def __init__(self, n_out: int, n_in: int, wt: int, w_local, rows: int = 1, group=None, align: int = 8,
                 host_counted: bool = False):
        import torch
        import torch.distributed as dist
        from . import capi
        self.capi, self.group, self.host_counted = capi, group, host_counted
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.n_out, self.n_in, self.wt, self.w_local = n_out, n_in, wt, w_local
        self.begin, self.count = row_range(n_out, self.world, self.rank, align)
        # two logits buffers and one flag word per peer (+ the device-side step count), in memory the
        # other processes map
        out_bytes, flag_bytes = rows * n_out * 4, 4 * (self.world + 2)
        self._bufs = _PeerBuffers(capi, [out_bytes, out_bytes, flag_bytes], group)
        self.out = [self._bufs.own[b].tensor((rows, n_out), torch.float32) for b in range(2)]
        self.flags = self._bufs.own[2].tensor((self.world + 2,), torch.int32)
        self.peer_out = [self._bufs.ptrs[0], self._bufs.ptrs[1]]
        self.peer_flags = self._bufs.ptrs[2]
        self.epoch = 0

    def close(self):
        self.out, self.flags = [], None
        self._bufs.close()

    def forward(self, x):
        """x: f32 [rows, n_in] on this GPU (the same on every rank). Returns the full [rows, n_out] row,
        complete in stream order. Steps alternate between the two buffers; with device-counted steps
        (the default) a pair of consecutive calls can be captured into a CUDA graph and replayed."""
        self.epoch += 1
        b = self.epoch & 1
        if self.host_counted:
            self.capi.gemv_allgather(self.peer_out[b], self.peer_flags, self.rank, self.epoch, self.begin, self.n_out, x,
                                     self.w_local, self.wt, self.count, self.n_in, wait_in_kernel=False)
            self.capi.wait_flags(self.flags, self.world, self.epoch)
        else:
            self.capi.gemv_allgather(self.peer_out[b], self.peer_flags, self.rank, 0, self.begin, self.n_out, x,
                                     self.w_local, self.wt, self.count, self.n_in, wait_in_kernel=True)
        return self.out[b]


class ShardedMoE:
    """Routed-expert FFN with the expert bank split over the ranks of ``group``.

    ``route_fn(logits) -> (ids, wts)`` is the replicated router; ``local_fn(x, ids, wts) ->
    [n_tok, n_embd]`` is the partial sum over the picks this rank holds. ``combine_fn(parts) ->
    [n_tok, n_embd]`` adds the gathered partials ``[world, n_tok, n_embd]`` in rank order. With
    ``exchange`` (a PeerSum) the all-gather and the sum are one kernel over NVLink peer stores instead.
    """

    def __init__(self, n_expert: int, route_fn: Callable, local_fn: Callable, combine_fn: Callable = None, group=None,
                 exchange: Callable = None, routed_fn: Callable = None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_expert = n_expert
        self.expert_base, self.n_local = expert_range(n_expert, self.world, self.rank)
        self.route_fn, self.local_fn = route_fn, local_fn
        self.combine_fn = combine_fn or sum_in_rank_order
        self.exchange = exchange          # part -> combined, replacing all-gather + combine_fn (PeerSum)
        self.routed_fn = routed_fn        # (x, logits) -> part, replacing route_fn + local_fn (one launch fewer)
        self._gather = None

    def forward(self, x, router_logits):
        import torch
        if self.routed_fn is not None:
            part = self.routed_fn(x, router_logits)
        else:
            ids, wts = self.route_fn(router_logits)
            part = self.local_fn(x, ids, wts)
        if self.world == 1:
            return part
        if self.exchange is not None:
            return self.exchange(part)
        if self._gather is None or self._gather.shape[1:] != part.shape or self._gather.device != part.device:
            self._flat = torch.empty((self.world * part.shape[0],) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
            self._gather = self._flat.view((self.world,) + tuple(part.shape))
        self.dist.all_gather_into_tensor(self._flat, part.contiguous(), group=self.group)
        return self.combine_fn(self._gather)

    def picks_per_rank(self, ids):
        """Histogram of the routed picks over the ranks (the load each GPU carries for this batch)."""
        flat = ids.reshape(-1).cpu()
        out = []
        for r in range(self.world):
            b, c = expert_range(self.n_expert, self.world, r)
            out.append(int(((flat >= b) & (flat < b + c)).sum()))
        return out


def sum_in_rank_order(parts):
    """((p0 + p1) + p2) + ... : a fixed association, identical on every rank and every run."""
    out = parts[0].clone()
    for r in range(1, parts.shape[0]):
        out += parts[r]
    return out


# ---- the CUDA library as the compute ------------------------------------------------------------

def cuda_head_fn(w_local, wt: int, count: int, n_in: int):
    """local_fn for ShardedHead over libkrk_cuda.so: w_local is this rank's [count, row_bytes] slice."""
    from . import capi

    def fn(x):
        return capi.gemv(x, w_local, wt, count, n_in)
    return fn


def cuda_moe_fns(bank, k: int):
    """(route_fn, local_fn, combine_fn) for ShardedMoE over libkrk_cuda.so; ``bank`` is this rank's
    capi.ExpertBank (expert_base / n_local already set to this rank's block)."""
    from . import capi

    def route_fn(logits):
        return capi.route(logits, k)

    def local_fn(x, ids, wts):
        return capi.moe_ffn(x, ids, wts, bank)

    def combine_fn(parts):
        return capi.sum_parts(parts)
    return route_fn, local_fn, combine_fn


def cuda_moe_routed_fn(bank, k: int):
    """routed_fn for ShardedMoE over libkrk_cuda.so: routing folded into the FFN's first kernel."""
    from . import capi

    def fn(x, logits):
        return capi.moe_ffn_routed(x, logits, k, bank)[0]
    return fn
