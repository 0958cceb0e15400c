"""Expert-parallel prefill: the 64 experts of every layer spread over the ranks of a process group, token rows
exchanged with all-to-all (NCCL over NVLink on GPUs; any torch.distributed backend for the host logic).

One layer, seen from a rank that holds `tokens` tokens (at most 2048 per call):

  plan      dest[pair] = owner of the pair's expert; the pairs sorted by destination (stable) give the send order
  pack      one BF16 row per pair in send order                                   (padra_ep_pack_rows)
  exchange  counts, then rows and their expert ids                                (all_to_all_single)
  experts   received rows grouped by expert, gate/up projections, SwiGLU, down    (padra_ep_group_rows,
                                                                                   padra_exl3_prefill_rows_launch)
  exchange  down rows back, same splits reversed: they arrive in send order
  combine   x[t] = B(x[t] + sum_s B(down * w)) reading pair p at row position[p]  (padra_ep_combine)

The reference serves one GPU and has no counterpart of this file; the arithmetic per row is that of its prefill path
(src/cuda/inference.cu:3896-3921).  The compute steps go through a backend object so that the exchange logic can be
run on CPU ranks (gloo) against a host implementation of the same three steps.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

EXPERTS, TOPK = 64, 8
MAX_ROWS = 4096 * TOPK  # rows one grouped-projection call takes (a rank may receive more rows than it sends)


def balanced_placement(popularity, world: int, replicas: int = 0, force: bool = False) -> np.ndarray:
    """owner[expert] for `world` ranks holding 64/world experts each: experts in order of falling popularity go to the
    rank with the least expected load that still has room (longest-processing-time-first).  Ties break towards the
    lower rank, so every rank computes the same table from the same popularity.

    replicas = k > 0: up to k of the most popular experts are held by a second rank as well (at most one extra expert's
    weights per rank: 3 MB at K4 2048/1024) and their pairs are split between the two ranks by token parity; such an
    entry is rank | (1 + second rank) << 8 (see owner_ranks).  Copies are added, most popular expert first, only while
    they lower the busiest rank's expected load.  With Zipf(1.1) routing on eight ranks the busiest rank's load drops
    from 1.155 times the mean to 1.05 with one copy."""
    popularity = np.asarray(popularity, dtype=np.float64)
    assert popularity.shape == (EXPERTS,) and EXPERTS % world == 0 and replicas >= 0
    replicas = min(replicas, world) if world > 1 else 0  # one extra expert per rank at most; nothing to copy to on one rank

    def place(split) -> np.ndarray:
        # items in order of falling share; a split expert is two items of half its popularity, the second of which takes
        # a rank's extra slot (one per rank, no room needed) and must not meet the first
        items = [(popularity[e] / 2 if e in split else popularity[e], int(e), 0) for e in range(EXPERTS)]
        items += [(popularity[e] / 2, int(e), 1) for e in split]
        items.sort(key=lambda item: (-item[0], item[1], item[2]))
        room, load, extra = np.full(world, EXPERTS // world), np.zeros(world), np.ones(world, dtype=bool)
        owner = np.empty(EXPERTS, dtype=np.int32)
        for share, e, second in items:
            if second:
                candidates = np.array([r for r in range(world) if r != (owner[e] & 0xff) and extra[r]])
            else:
                candidates = np.where(room > 0)[0]
            r = int(candidates[np.argmin(load[candidates])])
            load[r] += share
            if second:
                owner[e] |= (r + 1) << 8
                extra[r] = False
            else:
                owner[e], room[r] = r, room[r] - 1
        return owner

    best = place(())
    if world < 2:
        return best
    hottest = [int(e) for e in np.argsort(-popularity, kind="stable")]
    for k in range(1, replicas + 1):
        candidate = place(tuple(hottest[:k]))
        # force: keep the copies even where they do not help (to exercise the path on few ranks)
        if force or placement_load(popularity, candidate, world) < placement_load(popularity, best, world):
            best = candidate
        else:
            break
    return best


def owner_ranks(owner: np.ndarray):
    """(first rank, second rank or -1) per expert of an owner table."""
    owner = np.asarray(owner, dtype=np.int64)
    return owner & 0xff, ((owner >> 8) & 0xff) - 1


def placement_load(popularity, owner, world: int) -> float:
    """Expected load of the busiest rank over the mean, for pairs drawn with the given popularity."""
    popularity = np.asarray(popularity, dtype=np.float64)
    first, second = owner_ranks(owner)
    load = np.zeros(world)
    for e in range(EXPERTS):
        if second[e] >= 0:
            load[first[e]] += popularity[e] / 2
            load[second[e]] += popularity[e] / 2
        else:
            load[first[e]] += popularity[e]
    return float(load.max() / load.mean())


def contiguous_placement(world: int) -> np.ndarray:
    return (np.arange(EXPERTS) // (EXPERTS // world)).astype(np.int32)


@dataclass
class Plan:
    order: torch.Tensor       # [pairs] int32: pair sent as row j
    position: torch.Tensor    # [pairs] int32: row at which pair p comes back
    send_ids: torch.Tensor    # [pairs] int32: expert id of row j
    send_counts: torch.Tensor  # [world] int64: rows per destination


def make_plan(ids: torch.Tensor, owner: torch.Tensor, world: int) -> Plan:
    """ids [pairs] int32 expert ids in (token, slot) order; owner [64] on the same device."""
    flat = ids.reshape(-1).long()
    entry = owner[flat].long()
    second = (entry >> 8) & 0xff  # an expert held by two ranks: odd tokens' pairs go to the second
    odd_token = (torch.arange(flat.numel(), device=flat.device) >> 3) & 1
    dest = torch.where((second > 0) & (odd_token == 1), second - 1, entry & 0xff)
    order = torch.sort(dest, stable=True).indices
    position = torch.empty_like(order)
    position[order] = torch.arange(order.numel(), device=order.device)
    return Plan(order.to(torch.int32), position.to(torch.int32), flat[order].to(torch.int32),
                torch.bincount(dest, minlength=world))


class GroupExchange:
    """all-to-all over a torch.distributed process group.  The split sizes have to reach the host, which costs one
    synchronisation per layer call: the price of exact-size messages."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def counts(self, send_counts: torch.Tensor):
        recv = torch.empty_like(send_counts)
        dist.all_to_all_single(recv, send_counts, group=self.group)
        both = torch.stack([send_counts, recv]).cpu()
        return both[0].tolist(), both[1].tolist()

    def counts_many(self, send_counts: torch.Tensor):
        """send_counts [chunks][world] -> (send split lists, receive split lists), one host synchronisation."""
        recv = torch.empty_like(send_counts)
        for i in range(send_counts.shape[0]):
            dist.all_to_all_single(recv[i], send_counts[i], group=self.group)
        both = torch.stack([send_counts, recv]).cpu()
        return both[0].tolist(), both[1].tolist()

    def rows(self, send: torch.Tensor, send_splits, recv_splits) -> torch.Tensor:
        """Rows travel as bytes: every backend moves uint8, not every backend knows 16-bit integer types."""
        width = send[0].numel() * send.element_size() if send.dim() > 1 else send.element_size()
        recv = torch.empty((sum(recv_splits),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
        dist.all_to_all_single(recv.view(torch.uint8).reshape(-1, width), send.contiguous().view(torch.uint8).reshape(-1, width),
                               output_split_sizes=list(recv_splits), input_split_sizes=list(send_splits), group=self.group)
        return recv


class LoopbackHub:
    """Meeting point of LoopbackExchange ranks."""

    def __init__(self, world: int):
        import threading

        self.world = world
        self.barrier = threading.Barrier(world)
        self.slots = [None] * world


class LoopbackExchange:
    """The same interface with the ranks as threads of ONE process that share one device (and its default stream, so
    kernels run in launch order): lets the whole expert-parallel path run where only one GPU is to be had."""

    def __init__(self, hub: LoopbackHub, rank: int):
        self.hub, self.rank, self.world = hub, rank, hub.world

    def _swap(self, pieces):
        """pieces[destination] -> [piece from every source].  On a GPU the pieces come with an event of the sending
        thread's stream, which the receiving thread's stream waits for."""
        event = None
        if torch.cuda.is_available() and any(torch.is_tensor(p) and p.is_cuda for p in pieces):
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream())
        self.hub.slots[self.rank] = (pieces, event)
        self.hub.barrier.wait()
        got = []
        for source in range(self.world):
            theirs, their_event = self.hub.slots[source]
            if their_event is not None:
                torch.cuda.current_stream().wait_event(their_event)
            got.append(theirs[self.rank])
        self.hub.barrier.wait()
        return got

    def counts(self, send_counts: torch.Tensor):
        mine = [int(v) for v in send_counts.tolist()]
        return mine, self._swap(mine)

    def counts_many(self, send_counts: torch.Tensor):
        mine = [[int(v) for v in row] for row in send_counts.tolist()]
        theirs = self._swap([[row[d] for row in mine] for d in range(self.world)])  # theirs[source][chunk]
        return mine, [[theirs[source][c] for source in range(self.world)] for c in range(len(mine))]

    def rows(self, send: torch.Tensor, send_splits, recv_splits) -> torch.Tensor:
        as_bytes = send.contiguous().view(torch.uint8).reshape(send.shape[0], -1)
        got = self._swap(list(torch.split(as_bytes, list(send_splits))))
        assert [g.shape[0] for g in got] == list(recv_splits)
        return torch.cat(got).view(send.dtype).reshape((-1,) + tuple(send.shape[1:]))


class KernelBackend:
    """The three compute steps on the GPU through the C ABI."""

    def __init__(self, kernels):
        from . import binding as B

        self.k, self.B, self.lib = kernels, B, kernels.lib
        self.device = kernels.t.device
        self.hidden, self.inter = kernels.dims
        self._work = None

    def _workspace(self):
        if self._work is None:
            dev, h, i = self.device, self.hidden, self.inter
            self._work = dict(groups=torch.empty(EXPERTS * MAX_ROWS, dtype=torch.int32, device=dev),
                              counts=torch.empty(EXPERTS, dtype=torch.int32, device=dev),
                              gate=torch.empty((MAX_ROWS, i), dtype=torch.uint16, device=dev),
                              up=torch.empty((MAX_ROWS, i), dtype=torch.uint16, device=dev),
                              transformed=torch.empty((2 * MAX_ROWS, max(h, i)), dtype=torch.float16, device=dev))
        return self._work

    def plan(self, ids: torch.Tensor, owner: torch.Tensor, world: int) -> Plan:
        """make_plan in one kernel (padra_ep_plan); owner is int32 [64] on the device."""
        B, pairs, dev = self.B, ids.numel(), self.device
        order, position, send_ids = (torch.empty(pairs, dtype=torch.int32, device=dev) for _ in range(3))
        counts = torch.empty(world, dtype=torch.int64, device=dev)
        B.check(self.lib.padra_ep_plan(B.ptr(ids), B.ptr(owner), B.ptr(order), B.ptr(position), B.ptr(send_ids), B.ptr(counts),
                                       pairs, world, B.ptr(self.k.bad), B.stream_handle()), "padra_ep_plan")
        return Plan(order, position, send_ids, counts)

    def pack(self, plan: Plan, normalized: torch.Tensor) -> torch.Tensor:
        B, rows = self.B, plan.order.numel()
        packed = torch.empty((rows, self.hidden), dtype=torch.uint16, device=self.device)
        B.check(self.lib.padra_ep_pack_rows(B.ptr(normalized), B.ptr(plan.order), B.ptr(packed), rows, self.hidden,
                                            B.ptr(self.k.bad), B.stream_handle()), "padra_ep_pack_rows")
        return packed

    def experts(self, layer: int, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        B, w, k = self.B, self._workspace(), self.k
        total = rows.shape[0]
        down = torch.empty((total, self.hidden), dtype=torch.uint16, device=self.device)
        stream = B.stream_handle()
        for begin in range(0, total, MAX_ROWS):
            n = min(MAX_ROWS, total - begin)
            B.check(self.lib.padra_ep_group_rows(B.ptr(ids[begin:begin + n]), B.ptr(w["groups"]), B.ptr(w["counts"]), n, n,
                                                 B.ptr(k.bad), stream), "padra_ep_group_rows")
            # gate and up as one launch (one list of work items), then down
            B.check(self.lib.padra_exl3_prefill_rows_gate_up_launch(
                k.t.descriptors.data_ptr(), layer, B.ptr(w["groups"]), B.ptr(w["counts"]), n, n, B.ptr(rows[begin:begin + n]),
                B.ptr(w["gate"]), B.ptr(w["up"]), B.ptr(w["transformed"]), B.ptr(k.bad), stream, k.t.rate, self.hidden, self.inter),
                "padra_exl3_prefill_rows_gate_up_launch")
            B.check(self.lib.padra_exl3_prefill_rows_launch(
                k.t.descriptors.data_ptr(), layer, 2, B.ptr(w["groups"]), B.ptr(w["counts"]), n, n,
                B.ptr(rows[begin:begin + n]), B.ptr(down[begin:begin + n]), B.ptr(w["gate"]), B.ptr(w["up"]), B.ptr(k.table),
                B.ptr(w["transformed"]), B.ptr(k.bad), stream, k.t.rate, self.hidden, self.inter, 0, 0),
                "padra_exl3_prefill_rows_launch")
        return down

    def combine(self, plan: Plan, returned: torch.Tensor, routing: torch.Tensor, x: torch.Tensor) -> None:
        B, tokens = self.B, x.shape[0]
        B.check(self.lib.padra_ep_combine(B.ptr(x), B.ptr(returned), B.ptr(plan.position), B.ptr(routing), tokens,
                                          B.ptr(self.k.bad), 1, self.hidden, B.stream_handle()), "padra_ep_combine")


class PeerExchangePrefill:
    """The layer with the exchange done by the GPUs themselves: rows are stored straight into the owner rank's exchange
    block over NVLink, arrival is announced with epoch flags, and nothing returns to the host between the router and
    the combine (csrc/expert_parallel.cu).  `blocks` are this process's addresses of every rank's exchange block:
    symmetric memory of a process group (see `over_group`), or plain allocations when the ranks are threads that share
    one GPU (tests).  `between_phases` is called after the launches that announce rows and before the launch that waits
    for them; ranks that share ONE GPU pass a thread barrier there, so that in stream order every announcing kernel
    precedes every waiting kernel (kernels of one GPU must never wait for kernels launched later).
    `fused_return` lets the down projection's epilogue store its rows into the sources' blocks itself instead of a
    separate return kernel; measured at two GPUs it is a little slower (122 against 119 ms per batch), because the
    epilogue's 16-byte stores to scattered rows use NVLink less well than the return kernel's 512-byte ones."""

    MAX_GROUPED = 4096 * TOPK

    def __init__(self, kernels, owner, rank: int, world: int, cap: int, block: torch.Tensor, blocks, between_phases=None,
                 fused_return: bool = False, split_return: bool = True):
        import ctypes as C

        from . import binding as B

        self.k, self.B, self.lib = kernels, B, kernels.lib
        self.rank, self.world, self.cap = rank, world, cap
        self.device = kernels.t.device
        self.hidden, self.inter = kernels.dims
        self.block, self.between_phases, self.fused_return = block, between_phases, fused_return
        self.split_return = split_return
        offsets = (C.c_size_t * 6)()
        total = self.lib.padra_ep_exchange_bytes(world, cap, self.hidden, offsets)
        assert total and block.numel() >= total and block.dtype == torch.uint8
        self.offsets = list(offsets)
        self.bases = (C.c_ulonglong * 8)(*[int(b) for b in blocks], *([0] * (8 - world)))
        self.owner = torch.from_numpy(np.asarray(owner, dtype=np.int32)).to(self.device)
        dev, rows = self.device, world * cap
        self.groups = torch.empty(EXPERTS * self.MAX_GROUPED, dtype=torch.int32, device=dev)
        self.counts = torch.empty(EXPERTS, dtype=torch.int32, device=dev)
        self.gate = torch.empty((rows, self.inter), dtype=torch.uint16, device=dev)
        self.up = torch.empty((rows, self.inter), dtype=torch.uint16, device=dev)
        self.down = None if fused_return else torch.empty((rows, self.hidden), dtype=torch.uint16, device=dev)
        self.transformed = torch.empty((self.MAX_GROUPED, max(self.hidden, self.inter)), dtype=torch.float16, device=dev)
        self.transformed_up = torch.empty((self.MAX_GROUPED, self.hidden), dtype=torch.float16, device=dev)
        # gate and up as one launch: both parts' transformed rows, the second part's behind the first's
        self.merged_gate_up = True
        self.transformed_both = torch.empty((2 * min(rows, self.MAX_GROUPED), self.hidden), dtype=torch.float16, device=dev)
        self.backend = KernelBackend(kernels)
        self.epoch = 0
        self._side = None  # this engine's second stream (two engines may run side by side, each on its own pair of streams)

    def side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    @staticmethod
    def exchange_bytes(lib, world: int, cap: int, hidden: int) -> int:
        return lib.padra_ep_exchange_bytes(world, cap, hidden, None)

    @classmethod
    def over_group(cls, kernels, owner, cap: int, group=None, fused_return: bool = False, split_return: bool = True):
        """Exchange blocks in symmetric memory of a process group (one GPU per rank)."""
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings are all this needs
        import torch.distributed._symmetric_memory as symm_mem

        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        total = cls.exchange_bytes(kernels.lib, world, cap, kernels.dims[0])
        block = symm_mem.empty(total, dtype=torch.uint8, device=kernels.t.device)
        block.zero_()
        handle = symm_mem.rendezvous(block, group)
        torch.cuda.synchronize(kernels.t.device)
        dist.barrier(group)
        engine = cls(kernels, owner, rank, world, cap, block, [int(p) for p in handle.buffer_ptrs], fused_return=fused_return,
                     split_return=split_return)
        engine._handle = handle
        return engine

    def set_owner(self, owner) -> None:
        self.owner.copy_(torch.from_numpy(np.asarray(owner, dtype=np.int32)))

    def layer(self, layer: int, ids: torch.Tensor, routing: torch.Tensor, normalized: torch.Tensor, x: torch.Tensor,
              owner: torch.Tensor | None = None) -> None:
        """owner: int32 [64] on the device, if this layer's placement differs from the engine's."""
        B, lib, k = self.B, self.lib, self.k
        self.epoch += 1
        stream, bad = B.stream_handle(), B.ptr(k.bad)
        tokens, pairs = x.shape[0], ids.numel()
        geometry = (self.world, self.cap, self.hidden)
        base = self.block.data_ptr()
        plan = self.backend.plan(ids, self.owner if owner is None else owner, self.world)
        B.check(lib.padra_ep_dispatch(B.ptr(normalized), B.ptr(plan.order), B.ptr(plan.send_ids), B.ptr(plan.send_counts), self.bases,
                                      self.rank, self.world, self.cap, pairs, self.hidden, self.epoch, bad, stream), "padra_ep_dispatch")
        if self.between_phases:
            self.between_phases()
        B.check(lib.padra_ep_wait(base, 0, *geometry, self.epoch, bad, stream), "padra_ep_wait")
        B.check(lib.padra_ep_group_received(base, *geometry, B.ptr(self.groups), B.ptr(self.counts), self.MAX_GROUPED, bad, stream),
                "padra_ep_group_received")
        def project(part, target, transformed, on, blocks=(0, 0)):
            B.check(lib.padra_exl3_prefill_rows_launch(
                k.t.descriptors.data_ptr(), layer, part, B.ptr(self.groups), B.ptr(self.counts), self.MAX_GROUPED, self.world * self.cap,
                base + self.offsets[0], B.ptr(target), B.ptr(self.gate), B.ptr(self.up), B.ptr(k.table), B.ptr(transformed), bad,
                on, k.t.rate, self.hidden, self.inter, *blocks), "padra_exl3_prefill_rows_launch")

        main, side = torch.cuda.current_stream(), self.side_stream()
        if self.merged_gate_up:  # gate and up as one launch: one list of work items, one input transform
            B.check(lib.padra_exl3_prefill_rows_gate_up_launch(
                k.t.descriptors.data_ptr(), layer, B.ptr(self.groups), B.ptr(self.counts), self.MAX_GROUPED, self.world * self.cap,
                base + self.offsets[0], B.ptr(self.gate), B.ptr(self.up), B.ptr(self.transformed_both), bad, stream, k.t.rate,
                self.hidden, self.inter), "padra_exl3_prefill_rows_gate_up_launch")
        else:  # the up projection runs on a second stream beside the gate projection; both join before the down projection
            fork, join = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            project(1, self.up, self.transformed_up, side.cuda_stream)
            join.record(side)
            project(0, self.gate, self.transformed, stream)
            main.wait_event(join)
        if self.fused_return:  # the down projection's epilogue stores the rows into their sources' blocks itself
            B.check(lib.padra_ep_down_return(k.t.descriptors.data_ptr(), layer, B.ptr(self.groups), B.ptr(self.counts), self.MAX_GROUPED,
                                             B.ptr(self.gate), B.ptr(self.up), B.ptr(k.table), B.ptr(self.transformed), self.bases,
                                             self.rank, self.world, self.cap, self.epoch, bad, stream, k.t.rate, self.hidden, self.inter),
                    "padra_ep_down_return")
        elif self.split_return and self.world > 1:
            # the first half of the down rows' columns travels (second stream) while the second half is computed
            half = self.hidden // 256  # 128-output blocks per half
            sent, computed = torch.cuda.Event(), torch.cuda.Event()
            project(2, self.down, self.transformed, stream, (0, half))
            computed.record(main)
            side.wait_event(computed)
            B.check(lib.padra_ep_return(B.ptr(self.down), self.bases, self.rank, self.world, self.cap, self.hidden, self.epoch, bad,
                                        side.cuda_stream, 0, half * 128, 0), "padra_ep_return")
            sent.record(side)
            project(2, self.down, self.transformed, stream, (half, self.hidden // 128 - half))
            main.wait_event(sent)
            B.check(lib.padra_ep_return(B.ptr(self.down), self.bases, self.rank, self.world, self.cap, self.hidden, self.epoch, bad,
                                        stream, half * 128, self.hidden - half * 128, 1), "padra_ep_return")
        else:
            project(2, self.down, self.transformed, stream)
            B.check(lib.padra_ep_return(B.ptr(self.down), self.bases, self.rank, self.world, self.cap, self.hidden, self.epoch, bad,
                                        stream, 0, 0, 1), "padra_ep_return")
        if self.between_phases:
            self.between_phases()
        B.check(lib.padra_ep_wait(base, 1, *geometry, self.epoch, bad, stream), "padra_ep_wait")
        B.check(lib.padra_ep_combine(B.ptr(x), base + self.offsets[3], B.ptr(plan.position), B.ptr(routing), tokens, bad, 1, self.hidden,
                                     stream), "padra_ep_combine")


class ExpertParallelPrefill:
    """One MoE layer call for this rank's tokens; every rank of the group calls it together."""

    def __init__(self, backend, exchange, owner: np.ndarray):
        self.backend, self.exchange = backend, exchange
        self.owner_host = np.asarray(owner, dtype=np.int32)
        self._owner = {}
        self._comm_stream = None

    def owner_on(self, device, dtype=torch.int64) -> torch.Tensor:
        if (device, dtype) not in self._owner:
            self._owner[device, dtype] = torch.from_numpy(self.owner_host.astype(np.int64)).to(device=device, dtype=dtype)
        return self._owner[device, dtype]

    def _plan(self, ids: torch.Tensor) -> Plan:
        if hasattr(self.backend, "plan"):
            return self.backend.plan(ids, self.owner_on(ids.device, torch.int32), self.exchange.world)
        return make_plan(ids, self.owner_on(ids.device), self.exchange.world)

    def layer(self, layer: int, ids: torch.Tensor, routing: torch.Tensor, normalized: torch.Tensor, x: torch.Tensor) -> None:
        """ids/routing [tokens*8], normalized/x [tokens][hidden] (FP32 holding BF16 values); x updated in place."""
        ex = self.exchange
        plan = self._plan(ids)
        packed = self.backend.pack(plan, normalized)
        send_splits, recv_splits = ex.counts(plan.send_counts)
        rows = ex.rows(packed, send_splits, recv_splits)
        row_ids = ex.rows(plan.send_ids, send_splits, recv_splits)
        down = self.backend.experts(layer, rows, row_ids) if rows.shape[0] else rows
        returned = ex.rows(down, recv_splits, send_splits)
        self.backend.combine(plan, returned, routing, x)

    def layer_chunks(self, layer: int, chunks) -> None:
        """The same for several chunks [(ids, routing, normalized, x), ...] of this rank's tokens (every rank passes the
        same number of chunks), software-pipelined over two CUDA streams: while the experts of chunk i run, the rows of
        chunk i+1 arrive and the results of chunk i-1 leave.  One host synchronisation per call (the split sizes of
        all chunks travel together)."""
        ex, be = self.exchange, self.backend
        compute = torch.cuda.current_stream()
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=compute.device)
        comm = self._comm_stream
        n = len(chunks)
        plans, packed = [], []
        for ids, _, normalized, _ in chunks:
            plan = self._plan(ids)
            plans.append(plan)
            packed.append(be.pack(plan, normalized))
        ready = torch.cuda.Event()
        ready.record(compute)
        with torch.cuda.stream(comm):
            comm.wait_event(ready)
            send_splits, recv_splits = ex.counts_many(torch.stack([p.send_counts for p in plans]))  # the one host sync
        rows, row_ids, down, returned = [None] * n, [None] * n, [None] * n, [None] * n
        arrived = [torch.cuda.Event() for _ in range(n)]
        computed = [torch.cuda.Event() for _ in range(n)]
        back = [torch.cuda.Event() for _ in range(n)]

        def receive(i):
            with torch.cuda.stream(comm):
                rows[i] = ex.rows(packed[i], send_splits[i], recv_splits[i])
                row_ids[i] = ex.rows(plans[i].send_ids, send_splits[i], recv_splits[i])
                arrived[i].record(comm)
            for t in (rows[i], row_ids[i]):
                t.record_stream(compute)
            packed[i].record_stream(comm)
            plans[i].send_ids.record_stream(comm)

        def give_back(i):
            with torch.cuda.stream(comm):
                comm.wait_event(computed[i])
                returned[i] = ex.rows(down[i], recv_splits[i], send_splits[i])
                back[i].record(comm)
            returned[i].record_stream(compute)
            down[i].record_stream(comm)

        def combine(i):
            compute.wait_event(back[i])
            be.combine(plans[i], returned[i], chunks[i][1], chunks[i][3])

        receive(0)
        for i in range(n):
            if i + 1 < n:
                receive(i + 1)
            compute.wait_event(arrived[i])
            down[i] = be.experts(layer, rows[i], row_ids[i]) if rows[i].shape[0] else rows[i]
            computed[i].record(compute)
            give_back(i)
            if i > 0:
                combine(i - 1)
        combine(n - 1)
