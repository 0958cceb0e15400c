"""Expert-parallel prefill: placement, the exchange plan, and the whole layer over several ranks.

CPU: two gloo ranks run the layer with a host backend built on the oracle; every rank's result must equal the
oracle's single-process layer on that rank's tokens bit for bit (the exchange only moves rows).
GPU: the ranks are threads sharing one device (LoopbackExchange); results must equal the single-GPU prefill path."""
import threading

import numpy as np
import pytest
import torch

from oracle import exl3_oracle as O
from padra_b200 import expert_parallel as EP


def test_balanced_placement_fills_every_rank_and_balances():
    from padra_b200.experts import zipf_routing

    # popularity as a server would measure it: how many pairs of a 2048-token chunk each expert received
    ids, _ = zipf_routing(2048, seed=3, device="cpu")
    popularity = np.bincount(ids.reshape(-1).numpy(), minlength=64).astype(np.float64)
    for world in (1, 2, 4, 8):
        owner = EP.balanced_placement(popularity, world)
        assert np.bincount(owner, minlength=world).tolist() == [64 // world] * world
        load = np.array([popularity[owner == r].sum() for r in range(world)])
        contiguous = np.array([popularity[EP.contiguous_placement(world) == r].sum() for r in range(world)])
        assert load.max() <= contiguous.max() + 1e-12
        assert load.max() / load.mean() < 1.25
    assert (EP.balanced_placement(popularity, 8) == EP.balanced_placement(popularity, 8)).all()


def test_a_second_copy_of_the_hottest_expert_lowers_the_busiest_rank():
    from padra_b200.experts import zipf_routing

    ids, _ = zipf_routing(16384, seed=3, device="cpu")
    popularity = np.bincount(ids.reshape(-1).numpy(), minlength=64).astype(np.float64)
    for world in (2, 4, 8):
        exact = EP.balanced_placement(popularity, world)
        doubled = EP.balanced_placement(popularity, world, replicas=1)
        first, second = EP.owner_ranks(doubled)
        hottest = int(np.argmax(popularity))
        assert np.bincount(first, minlength=world).tolist() == [64 // world] * world
        assert EP.placement_load(popularity, doubled, world) <= EP.placement_load(popularity, exact, world) + 1e-12
        if world == 8:  # the copy is only made where it helps
            assert (second >= 0).sum() == 1 and second[hottest] >= 0 and second[hottest] != first[hottest]
    assert (EP.balanced_placement(popularity, 1, replicas=2) == 0).all()  # one rank: nothing to copy to
    two = EP.balanced_placement(popularity, 8, replicas=2)
    assert ((two >> 8) > 0).sum() == 2 and len(set(((two >> 8) & 0xff)[(two >> 8) > 0])) == 2  # two copies on two different ranks
    assert EP.placement_load(popularity, two, 8) < EP.placement_load(popularity, EP.balanced_placement(popularity, 8, replicas=1), 8)
    assert EP.placement_load(popularity, EP.balanced_placement(popularity, 8), 8) > 1.12
    assert EP.placement_load(popularity, EP.balanced_placement(popularity, 8, replicas=1), 8) < 1.06
    # the plan sends the even tokens' pairs of that expert to the first rank and the odd tokens' to the second
    owner = EP.balanced_placement(popularity, 8, replicas=1)
    first, second = EP.owner_ranks(owner)
    chunk = ids[:256].reshape(-1)
    plan = EP.make_plan(chunk, torch.from_numpy(owner.astype(np.int64)), 8)
    dest = np.repeat(np.arange(8), plan.send_counts.numpy())
    for row, pair in enumerate(plan.order.numpy()):
        e = int(chunk[pair])
        want = second[e] if second[e] >= 0 and (pair >> 3) & 1 else first[e]
        assert dest[row] == want


def test_plan_is_a_stable_sort_by_destination():
    g = torch.Generator().manual_seed(5)
    ids = torch.stack([torch.randperm(64, generator=g)[:8] for _ in range(40)]).to(torch.int32)
    owner = torch.from_numpy(EP.contiguous_placement(4).astype(np.int64))
    plan = EP.make_plan(ids.reshape(-1), owner, 4)
    dest = owner[ids.reshape(-1).long()]
    sent = dest[plan.order.long()]
    assert (sent[1:] >= sent[:-1]).all()
    for r in range(4):
        mine = plan.order[sent == r]
        assert (mine[1:] > mine[:-1]).all()  # stable: ascending pair order inside a destination
    assert plan.send_counts.tolist() == torch.bincount(dest, minlength=4).tolist()
    assert (plan.order[plan.position.long()] == torch.arange(320, dtype=torch.int32)).all()
    assert (plan.send_ids == ids.reshape(-1)[plan.order.long()]).all()


class HostBackend:
    """pack / experts / combine on the CPU through the oracle (test infrastructure)."""

    def __init__(self, oracle, host, hidden, inter, rate):
        self.o, self.host, self.hidden, self.inter, self.rate = oracle, host, hidden, inter, rate
        self.silu = oracle.silu_table().astype(np.uint32)

    @staticmethod
    def bits(x):
        return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)

    @staticmethod
    def values(b):
        return (np.asarray(b).astype(np.uint32) << 16).view(np.float32)

    def pack(self, plan, normalized):
        rows = normalized.numpy()[plan.order.numpy() >> 3]
        return torch.from_numpy(self.bits(rows).view(np.int16))

    def experts(self, layer, rows, ids):
        x = self.values(rows.numpy().view(np.uint16))
        out = np.empty((x.shape[0], self.hidden), np.float32)
        for r, e in enumerate(ids.tolist()):
            m = [self.o.matrix(*self.host.get(layer, e, part), *((self.hidden, self.inter) if part == 2 else (self.inter, self.hidden)),
                               self.rate) for part in range(3)]
            gate, _ = self.o.linear(m[0], x[r])
            up, _ = self.o.linear(m[1], x[r])
            act = O.bf16_round(self.values(self.silu[self.bits(gate)]) * up)
            out[r], _ = self.o.linear(m[2], act)
        return torch.from_numpy(self.bits(out).view(np.int16))

    def combine(self, plan, returned, routing, x):
        down = self.values(returned.numpy().view(np.uint16))[plan.position.numpy()].reshape(x.shape[0], 8, self.hidden)
        w = routing.numpy().reshape(-1, 8)
        total = np.zeros_like(x.numpy())
        for s in range(8):
            total = O.bf16_round(total + O.bf16_round(down[:, s] * w[:, s:s + 1]))
        x.copy_(torch.from_numpy(O.bf16_round(x.numpy() + total)))


def _inputs(oracle, rank, tokens, hidden):
    rng = np.random.default_rng(100 + rank)
    x = O.bf16_round(rng.standard_normal((tokens, hidden)).astype(np.float32))
    ids, w, bad = oracle.route(O.bf16_round(rng.standard_normal((tokens, 64)).astype(np.float32)))
    assert not bad
    return x, ids, w


def _gloo_rank(rank, world, port, results):
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        oracle = O.COracle()
        hidden, inter, tokens = 256, 128, 6
        host = O.HostMatrices(1, hidden, inter, 4, seed=21)
        x, ids, w = _inputs(oracle, rank, tokens, hidden)
        popularity = np.arange(1, 65, dtype=np.float64) ** -1.1
        owner = EP.balanced_placement(popularity, world)
        owner[0] |= ((int(owner[0]) + 1) % world + 1) << 8  # expert 0 held by both ranks: odd tokens' pairs go to the second
        ep = EP.ExpertParallelPrefill(HostBackend(oracle, host, hidden, inter, 4), EP.GroupExchange(), owner)
        got = torch.from_numpy(x.copy())
        ep.layer(0, torch.from_numpy(ids.reshape(-1)), torch.from_numpy(w.reshape(-1)), torch.from_numpy(x), got)
        want, bad = oracle.moe_layer(host.table, 0, ids, w, x, hidden, inter)
        results.put((rank, bool(not bad and np.array_equal(got.numpy(), want)), float(np.abs(got.numpy() - want).max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_gloo_ranks_equal_the_single_process_layer():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29650 + (threading.get_native_id() % 200)
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    got = sorted(results.get(timeout=5) for _ in range(2))
    assert [g[:2] for g in got] == [(0, True), (1, True)], got


@pytest.mark.gpu
@pytest.mark.parametrize("world,chunks", [(2, 1), (4, 1), (2, 3), (8, 2)])
def test_ranks_on_one_gpu_equal_the_single_gpu_prefill(oracle, gpu, world, chunks):
    from padra_b200.experts import ExpertKernels, ExpertTable

    hidden, inter, tokens, rate = 512, 256, 40, 4
    host = O.HostMatrices(1, hidden, inter, rate, seed=33)
    table = ExpertTable(1, hidden, inter, rate, gpu).fill_from_host(host)
    hub = EP.LoopbackHub(world)
    popularity = np.arange(1, 65, dtype=np.float64) ** -1.1
    owner = EP.balanced_placement(popularity, world)
    if world > 2:  # a second copy of expert 0 on another rank
        owner[0] |= ((int(owner[0]) + 1) % world + 1) << 8
    kernels = [ExpertKernels(table) for _ in range(world)]
    tokens *= chunks
    inputs = [_inputs(oracle, r, tokens, hidden) for r in range(world)]
    outputs, errors = [None] * world, []

    def run(rank):
        try:
            torch.cuda.set_device(gpu)
            x, ids, w = inputs[rank]
            ep = EP.ExpertParallelPrefill(EP.KernelBackend(kernels[rank]), EP.LoopbackExchange(hub, rank), owner)
            got = torch.from_numpy(x.copy()).to(gpu)
            dids, dw, dx = torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu), torch.from_numpy(x).to(gpu)
            if chunks == 1:
                ep.layer(0, dids, dw, dx, got)
            else:  # the pipelined form: several chunks, two streams
                n = tokens // chunks
                ep.layer_chunks(0, [(dids[8 * n * c:8 * n * (c + 1)], dw[8 * n * c:8 * n * (c + 1)], dx[n * c:n * (c + 1)],
                                     got[n * c:n * (c + 1)]) for c in range(chunks)])
            outputs[rank] = got
        except Exception as e:  # a failing rank must not leave the others at the barrier
            errors.append(e)
            hub.barrier.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    torch.cuda.synchronize()
    for rank in range(world):
        x, ids, w = inputs[rank]
        want = torch.from_numpy(x.copy()).to(gpu)
        kernels[rank].prefill_layer(0, torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu),
                                    torch.from_numpy(x).to(gpu), want, tokens)
        torch.cuda.synchronize()
        assert kernels[rank].bad_flag() == 0
        assert np.array_equal(outputs[rank].cpu().numpy(), want.cpu().numpy()), f"rank {rank} differs from the single-GPU path"


@pytest.mark.gpu
@pytest.mark.parametrize("world,fused_return,split_return", [(2, True, False), (4, False, True), (2, False, True), (2, False, False)])
def test_peer_memory_exchange_on_one_gpu_equals_the_single_gpu_prefill(oracle, gpu, world, fused_return, split_return):
    """The exchange over peer memory with the ranks as threads of one process: every rank's block is a plain allocation
    of the shared GPU, and a thread barrier between the announcing and the waiting launches keeps the stream order that
    a single GPU needs.  Three layer calls in a row reuse the blocks."""
    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable

    hidden, inter, tokens, rate, layers = 512, 256, 48, 4, 3
    host = O.HostMatrices(layers, hidden, inter, rate, seed=35)
    table = ExpertTable(layers, hidden, inter, rate, gpu).fill_from_host(host)
    lib = B.load()
    cap = tokens * 8
    total = EP.PeerExchangePrefill.exchange_bytes(lib, world, cap, hidden)
    blocks = [torch.zeros(total, dtype=torch.uint8, device=gpu) for _ in range(world)]
    popularity = np.arange(1, 65, dtype=np.float64) ** -1.1
    owner = EP.balanced_placement(popularity, world)
    if split_return:  # expert 0 (in every token's top-8 here more often than any other) held by two ranks
        owner[0] |= ((int(owner[0]) + 1) % world + 1) << 8
    kernels = [ExpertKernels(table) for _ in range(world)]
    inputs = [_inputs(oracle, r, tokens, hidden) for r in range(world)]
    barrier = threading.Barrier(world)
    outputs, errors = [None] * world, []
    torch.cuda.synchronize()

    def run(rank):
        try:
            torch.cuda.set_device(gpu)
            x, ids, w = inputs[rank]
            engine = EP.PeerExchangePrefill(kernels[rank], owner, rank, world, cap, blocks[rank], [b.data_ptr() for b in blocks],
                                            between_phases=barrier.wait, fused_return=fused_return, split_return=split_return)
            got = torch.from_numpy(x.copy()).to(gpu)
            dids, dw, dx = torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu), torch.from_numpy(x).to(gpu)
            for layer in range(layers):
                engine.layer(layer, dids, dw, dx, got)
            outputs[rank] = got
        except Exception as e:
            errors.append(e)
            barrier.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    torch.cuda.synchronize()
    for rank in range(world):
        x, ids, w = inputs[rank]
        want = torch.from_numpy(x.copy()).to(gpu)
        dids, dw, dx = torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu), torch.from_numpy(x).to(gpu)
        for layer in range(layers):
            kernels[rank].prefill_layer(layer, dids, dw, dx, want, tokens)
        torch.cuda.synchronize()
        assert kernels[rank].bad_flag() == 0
        assert np.array_equal(outputs[rank].cpu().numpy(), want.cpu().numpy()), f"rank {rank} differs from the single-GPU path"


@pytest.mark.gpu
@pytest.mark.parametrize("world,tokens,replicas", [(1, 8, 0), (2, 333, 1), (8, 2048, 0), (8, 2048, 1)])
def test_plan_kernel_equals_the_host_plan(gpu, world, tokens, replicas):
    from padra_b200.experts import ExpertKernels, ExpertTable, zipf_routing

    table = ExpertTable(1, 256, 128, 4, gpu).fill_random(1)
    backend = EP.KernelBackend(ExpertKernels(table))
    ids, _ = zipf_routing(tokens, seed=world, device=gpu)
    popularity = np.bincount(ids.reshape(-1).cpu().numpy(), minlength=64)
    owner = EP.balanced_placement(popularity, world, replicas=replicas)
    want = EP.make_plan(ids.reshape(-1), torch.from_numpy(owner.astype(np.int64)).to(gpu), world)
    got = backend.plan(ids.reshape(-1), torch.from_numpy(owner).to(gpu), world)
    torch.cuda.synchronize()
    assert torch.equal(got.order, want.order) and torch.equal(got.position, want.position)
    assert torch.equal(got.send_ids, want.send_ids) and got.send_counts.tolist() == want.send_counts.tolist()


def test_exchange_block_layout_is_consistent():
    """Host-only: the byte layout of an exchange block (no GPU needed, the function only computes sizes)."""
    import ctypes as C

    from padra_b200 import binding as B

    lib = B.load()
    offsets = (C.c_size_t * 6)()
    world, cap, hidden = 8, 16384, 2048
    total = lib.padra_ep_exchange_bytes(world, cap, hidden, offsets)
    rows, ids, meta, returned, arrived, came_back = list(offsets)
    assert rows == 0 and ids == world * cap * hidden * 2                      # received rows first, BF16
    assert meta - ids >= world * cap * 4 and returned - meta >= world * 16   # ids, then one 16-byte record per source
    assert arrived - returned >= cap * hidden * 2 and came_back - arrived >= world * 4
    assert total > came_back and all(o % 256 == 0 for o in offsets) and total % 256 == 0
    assert lib.padra_ep_exchange_bytes(9, cap, hidden, None) == 0             # at most eight ranks
    assert lib.padra_ep_exchange_bytes(world, cap, 100, None) == 0            # hidden must be a multiple of 128
    assert lib.padra_ep_exchange_bytes(world, 4, hidden, None) == 0           # at least one token's pairs


@pytest.mark.gpu
def test_exchange_wait_gives_up_and_leaves_the_stream_usable():
    """padra_ep_wait on a block that nobody will ever announce into: after the (shortened) time limit the kernel raises
    the error flag and returns; the next launch on the stream runs as usual.  This is the path a rank takes when a peer
    never sends -- made here without any peer, so nothing on the GPU hangs or faults."""
    import ctypes as C
    import time

    from padra_b200 import binding as B

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = B.load()
    dev = torch.device("cuda:0")
    world, cap, hidden = 2, 64, 256
    total = lib.padra_ep_exchange_bytes(world, cap, hidden, None)
    block = torch.zeros(total, dtype=torch.uint8, device=dev)  # no flag ever carries epoch 1
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    assert lib.padra_ep_set_wait_limit_ms(0) == B.INVALID_ARGUMENT
    assert lib.padra_ep_set_wait_limit_ms(50) == B.OK
    try:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        assert lib.padra_ep_wait(block.data_ptr(), 0, world, cap, hidden, 1, bad.data_ptr(), B.stream_handle()) == B.OK
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert int(bad.item()) == 1, "an expired wait must raise the error flag"
        assert 0.04 <= waited < 1.0, f"the wait took {waited:.3f} s against a 50 ms limit"
        # the stream goes on: an ordinary launch of the library and a torch kernel both complete
        table = torch.empty(65536, dtype=torch.uint16, device=dev)
        assert lib.padra_exl3_silu_build(table.data_ptr(), B.stream_handle()) == B.OK
        torch.cuda.synchronize()
        assert int(table.view(torch.int16)[0x3F80].item()) != 0  # silu(1.0) is not zero
        # a flag that is there is seen at once
        offsets = (C.c_size_t * 6)()
        lib.padra_ep_exchange_bytes(world, cap, hidden, offsets)
        block[offsets[4]:offsets[4] + 4 * world].view(torch.int32).fill_(7)
        bad.zero_()
        assert lib.padra_ep_wait(block.data_ptr(), 0, world, cap, hidden, 7, bad.data_ptr(), B.stream_handle()) == B.OK
        torch.cuda.synchronize()
        assert int(bad.item()) == 0
    finally:
        assert lib.padra_ep_set_wait_limit_ms(2000) == B.OK
