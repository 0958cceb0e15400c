"""GPU parity tests of the prefill-side entry points (grouping, tile schedule, projections, combine)."""
import numpy as np
import pytest
import torch

from oracle import exl3_oracle as O
from tests.helpers import assert_close_rows, bf16_bits_to_f32, u16
from tests.test_gpu_decode import make, needs_ref, routed_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens", [4, 33, 257, 2048])
def test_group_and_schedule_match_oracle(oracle, gpu, tokens):
    from padra_b200.experts import zipf_routing

    _, table, k = make(1, 256, 128, 4, 71, gpu)
    ids, _ = zipf_routing(tokens, seed=tokens, device=gpu)
    groups, counts, tiles, tile_count = k.group_and_schedule(ids.reshape(-1), tokens)
    h_ids = ids.cpu().numpy()
    og, oc, bad = oracle.group(h_ids, tokens)
    assert not bad
    assert (counts.cpu().numpy() == oc).all()
    g = groups.cpu().numpy().reshape(64, tokens)
    og = og.reshape(64, tokens)
    for e in range(64):
        assert (g[e, : oc[e]] == og[e, : oc[e]]).all()
    ot, bad = oracle.schedule(oc, tokens)
    assert not bad
    n = int(tile_count.item())
    assert n == len(ot) and (tiles.cpu().numpy()[:n] == ot).all()
    assert k.bad_flag() == 0


def test_group_rejects_duplicate_expert(gpu):
    _, table, k = make(1, 256, 128, 4, 73, gpu)
    ids = torch.arange(8, dtype=torch.int32, device=gpu).repeat(4)
    ids[9] = 0  # token 1 uses expert 0 twice
    k.group_and_schedule(ids, 4)
    torch.cuda.synchronize()
    assert k.bad_flag() == 1


@pytest.mark.parametrize("tensor_memory", [False, True])
@pytest.mark.parametrize("rate", [3, 4, 6])
@pytest.mark.parametrize("tokens", [4, 37])
def test_prefill_layer_vs_oracle(oracle, gpu, rate, tokens, tensor_memory):
    hidden, inter = 256, 128
    host, table, k = make(1, hidden, inter, rate, 79, gpu)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 15 + tokens)
    want, bad, (cg, cu, ca, cd) = oracle.moe_layer(host.table, 0, ids, w, x, hidden, inter, capture=True)
    assert not bad
    dx = torch.from_numpy(x).to(gpu)
    xs = dx.clone()
    gate, up, down = k.prefill_layer(0, torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu),
                                     dx, xs, tokens, tensor_memory=tensor_memory)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert_close_rows(bf16_bits_to_f32(u16(gate)), cg, "prefill gate")
    assert_close_rows(bf16_bits_to_f32(u16(up)), cu, "prefill up")
    assert_close_rows(bf16_bits_to_f32(u16(down)), cd, "prefill down", chained=True)  # fed by its own gate/up
    assert_close_rows(xs.cpu().numpy(), want, "prefill layer", chained=True)


def test_tensor_memory_gemm_large_imbalanced_chunk(oracle, gpu):
    """600 tokens with Zipf routing: experts with more than 256 pairs (several token tiles) and with very few, both
    prefill kernels against each other and, for a sample of pairs, against the oracle."""
    from padra_b200.experts import bf16_values, zipf_routing

    hidden, inter, tokens = 512, 384, 600
    host, table, k = make(1, hidden, inter, 4, 211, gpu)
    ids, w = zipf_routing(tokens, seed=3, device=gpu)
    g = torch.Generator(device=gpu)
    g.manual_seed(2)
    dx = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    xa, xb = dx.clone(), dx.clone()
    ga, ua, da = (t.clone() for t in k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xa, tokens, tensor_memory=True))
    gb, ub, db = k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xb, tokens, tensor_memory=False)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert_close_rows(bf16_bits_to_f32(u16(ga)), bf16_bits_to_f32(u16(gb)), "gate: tensor-memory vs small-tile kernel")
    assert_close_rows(bf16_bits_to_f32(u16(ua)), bf16_bits_to_f32(u16(ub)), "up: tensor-memory vs small-tile kernel")
    assert_close_rows(xa.cpu().numpy(), xb.cpu().numpy(), "layer: tensor-memory vs small-tile kernel", chained=True)
    h_ids, h_x = ids.cpu().numpy(), dx.cpu().numpy()
    gate = bf16_bits_to_f32(u16(ga))
    for pair in (0, 777, 4799):
        e = int(h_ids.reshape(-1)[pair])
        data, suh, svh = host.get(0, e, 0)
        want, bad = oracle.linear(oracle.matrix(data, suh, svh, inter, hidden, 4), h_x[pair // 8])
        assert not bad
        assert_close_rows(gate[pair][None], want[None], f"gate row of pair {pair} vs oracle")


@pytest.mark.parametrize("rate,hidden,inter,tokens", [(4, 512, 384, 600), (3, 256, 128, 37), (6, 384, 896, 200)])
def test_gate_and_up_in_one_launch_equal_the_two_launches(gpu, rate, hidden, inter, tokens):
    """The merged launch only reorders work items: every row of gate, up, down and x is bit-equal to the rows of the
    part-by-part call sequence (inter 896 = seven output blocks: an item with a single block in each part)."""
    from padra_b200.experts import bf16_values, zipf_routing

    host, table, k = make(1, hidden, inter, rate, 77, gpu)
    ids, w = zipf_routing(tokens, seed=5, device=gpu)
    g = torch.Generator(device=gpu)
    g.manual_seed(9)
    dx = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    xa, xb = dx.clone(), dx.clone()
    ga, ua, da = (t.clone() for t in k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xa, tokens, merged=True))
    gb, ub, db = k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xb, tokens, merged=False)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert torch.equal(ga, gb) and torch.equal(ua, ub) and torch.equal(da, db) and torch.equal(xa, xb)


def test_routed_chunk_in_six_launches_equals_the_step_by_step_path(gpu):
    """prefill_chunk (routing + grouping + schedule in one launch, merged gate+up, reused buffers) against route() followed
    by prefill_layer's separate grouping and scheduling launches; twice, so that the second call meets used buffers."""
    from padra_b200.experts import bf16_values, zipf_logits

    hidden, inter, tokens = 512, 384, 600
    host, table, k = make(1, hidden, inter, 4, 19, gpu)
    g = torch.Generator(device=gpu)
    g.manual_seed(4)
    for seed in (1, 2):
        logits = zipf_logits(tokens, seed=seed, device=gpu)
        dx = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
        xa, xb = dx.clone(), dx.clone()
        ids, w = k.route(logits)
        k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xa, tokens, merged=False)
        ids2, w2 = k.prefill_chunk(0, logits, dx, xb, tokens)
        torch.cuda.synchronize()
        assert k.bad_flag() == 0
        assert torch.equal(ids, ids2) and torch.equal(w, w2) and torch.equal(xa, xb)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=64)
    assert counts.max() > 4 * counts.min()  # the logits are skewed as asked


def test_prefill_matches_decode_path(oracle, gpu):
    """The same tokens through the prefill entry points and through the decode layer call."""
    hidden, inter, tokens = 512, 256, 16
    host, table, k = make(1, hidden, inter, 4, 83, gpu)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 17)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dw = torch.from_numpy(w.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    a, b = dx.clone(), dx.clone()
    k.prefill_layer(0, dids, dw, dx, a, tokens)
    k.moe_decode_layer(0, dids, dw, dx, b, tokens)
    assert_close_rows(a.cpu().numpy(), b.cpu().numpy(), "prefill vs decode path", chained=True)
    assert k.bad_flag() == 0


def test_prefill_refuses_fewer_than_four_tokens(gpu):
    from padra_b200 import binding as B

    _, table, k = make(1, 256, 128, 4, 89, gpu)
    st = k.lib.padra_exl3_prefill_launch(table.descriptors.data_ptr(), 0, 0, *([None] * 11), 3, None, None, None, 0, 4, 256, 128)
    assert st == B.INVALID_ARGUMENT


@needs_ref
@pytest.mark.parametrize("rate", [3, 4, 6])
def test_against_reference_prefill_kernels_mellum_dims(oracle, gpu, rate):
    """Reference launchers (K4: exl3_transport_async64::Launch, K3/K6: exl3_packed_activations::Launch) with the
    reference's Group/Schedule, vs this library, at hidden 2304 / intermediate 896, 64 tokens, Zipf routing."""
    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable, bf16_values, zipf_routing

    hidden, inter, tokens = 2304, 896, 64
    pairs = tokens * 8
    table = ExpertTable(1, hidden, inter, rate, gpu).fill_random(200 + rate)
    k = ExpertKernels(table)
    ref = O.RefKernels()
    ids, w = zipf_routing(tokens, seed=5, device=gpu)
    g = torch.Generator(device=gpu)
    g.manual_seed(1)
    dx = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    s = B.stream_handle()
    D = table.descriptors.data_ptr()
    groups = torch.zeros(64 * tokens, dtype=torch.int32, device=gpu)
    counts = torch.zeros(64, dtype=torch.int32, device=gpu)
    tiles = torch.zeros((pairs // 32 + 65, 3), dtype=torch.int32, device=gpu)
    tile_count = torch.zeros(1, dtype=torch.int32, device=gpu)
    ref.ref_group(B.ptr(ids), B.ptr(groups), B.ptr(counts), tokens, B.ptr(bad), s)
    ref.ref_schedule(B.ptr(counts), B.ptr(tiles), B.ptr(tile_count), tokens, B.ptr(bad), s)
    ours = k.group_and_schedule(ids.reshape(-1), tokens)
    n = int(tile_count.item())
    assert torch.equal(ours[1], counts) and int(ours[3].item()) == n and torch.equal(ours[2][:n], tiles[:n])
    rgate = torch.zeros((pairs, inter), dtype=torch.int16, device=gpu)
    rup = torch.zeros((pairs, inter), dtype=torch.int16, device=gpu)
    rdown = torch.zeros((pairs, hidden), dtype=torch.int16, device=gpu)
    work = torch.zeros((pairs, hidden), dtype=torch.float16, device=gpu)
    for part, target in ((0, rgate), (1, rup), (2, rdown)):
        ref.ref_prefill_launch(D, 0, part, B.ptr(ids), B.ptr(groups), B.ptr(counts), B.ptr(tiles), B.ptr(tile_count), B.ptr(dx),
                               B.ptr(target), B.ptr(rgate), B.ptr(rup), B.ptr(k.table), B.ptr(work), tokens, B.ptr(bad), s, rate)
    rx = dx.clone()
    ref.ref_combine_packed(B.ptr(rx), B.ptr(rdown), B.ptr(w), tokens, B.ptr(bad), 1, s)
    torch.cuda.synchronize()
    assert int(bad.item()) == 0
    xs = dx.clone()
    gate, up, down = k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xs, tokens)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert_close_rows(bf16_bits_to_f32(u16(gate)), bf16_bits_to_f32(u16(rgate)), "gate vs reference prefill")
    assert_close_rows(bf16_bits_to_f32(u16(up)), bf16_bits_to_f32(u16(rup)), "up vs reference prefill")
    assert_close_rows(bf16_bits_to_f32(u16(down)), bf16_bits_to_f32(u16(rdown)), "down vs reference prefill", chained=True)
    assert_close_rows(xs.cpu().numpy(), rx.cpu().numpy(), "layer vs reference prefill", chained=True)


@pytest.mark.parametrize("rate", [3, 4, 6])
def test_prefill_maximum_chunk_with_empty_and_full_experts(oracle, gpu, rate):
    """The largest chunk the entry points take (2048 tokens), routed so that eight experts receive every token (2048
    pairs each: eight full 256-token items per output block) and fifty-six experts receive none; both prefill kernels
    against each other on the whole layer and, for pairs of the first, a middle and the last item, against the oracle."""
    from padra_b200.experts import bf16_values

    hidden, inter, tokens = 256, 128, 2048
    host, table, k = make(1, hidden, inter, rate, 300 + rate, gpu)
    chosen = torch.tensor([1, 5, 12, 20, 33, 47, 58, 63], dtype=torch.int32, device=gpu)
    ids = chosen.repeat(tokens)
    g = torch.Generator(device=gpu)
    g.manual_seed(9)
    w = torch.rand((tokens, 8), device=gpu, generator=g) + 0.1
    w = bf16_values(w / w.sum(dim=-1, keepdim=True)).reshape(-1)
    dx = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    xa, xb = dx.clone(), dx.clone()
    ga, ua, da = (t.clone() for t in k.prefill_layer(0, ids, w, dx, xa, tokens, tensor_memory=True))
    k.prefill_layer(0, ids, w, dx, xb, tokens, tensor_memory=False)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    # two summation orders on a chained result, half a million elements: compared in the row 2-norm (1e-2) and element
    # by element against max(|ref|, rms) (3e-2); the worst single element of 2048 rows sits at the 1e-2 line itself
    a, b = xa.cpu().numpy().astype(np.float64), xb.cpu().numpy().astype(np.float64)
    assert (np.linalg.norm(a - b, axis=1) <= 1e-2 * np.linalg.norm(b, axis=1)).all()
    floor = np.maximum(np.abs(b), np.sqrt((b ** 2).mean(axis=1, keepdims=True)))
    assert (np.abs(a - b) <= 3e-2 * floor).all()
    h_x, gate = dx.cpu().numpy(), bf16_bits_to_f32(u16(ga))
    for pair in (0, 8 * 1000 + 3, 8 * 2047 + 7):
        e = int(chosen[pair % 8])
        data, suh, svh = host.get(0, e, 0)
        want, bad = oracle.linear(oracle.matrix(data, suh, svh, inter, hidden, rate), h_x[pair // 8])
        assert not bad
        assert_close_rows(gate[pair][None], want[None], f"gate row of pair {pair} vs oracle")


def test_prefill_smallest_chunk(oracle, gpu):
    """Four tokens, the fewest the prefill launchers take: 32 pairs, most experts empty, against the oracle's layer."""
    hidden, inter, tokens = 256, 128, 4
    host, table, k = make(1, hidden, inter, 4, 97, gpu)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 23)
    dids, dw, dx = torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu), torch.from_numpy(x).to(gpu)
    got = dx.clone()
    k.prefill_layer(0, dids, dw, dx, got, tokens)
    torch.cuda.synchronize()
    want, bad = oracle.moe_layer(host.table, 0, ids, w, x, hidden, inter)
    assert not bad and k.bad_flag() == 0
    assert_close_rows(got.cpu().numpy(), want, "four-token prefill layer vs oracle", chained=True)


@pytest.mark.parametrize("hidden,inter,tokens,rate", [
    (128, 128, 5, 4),      # one output block per part, two 64-input stages: fewer stages than the look-ahead
    (384, 256, 129, 3),    # three blocks in the down part (odd: the last item has a single block)
    (256, 384, 300, 6),    # three blocks in gate/up, experts with one and with several token tiles
    (640, 128, 1111, 4),   # five blocks, long K for gate/up and two stages for down
])
def test_tensor_memory_gemm_odd_shapes(oracle, gpu, hidden, inter, tokens, rate):
    """Shapes that exercise the item list's corners: odd numbers of output blocks, very short K, token tiles of every
    filling.  The tensor-memory GEMM against the small-tile kernel (an independent implementation) on gate, up and the
    whole layer, and against the oracle for a few pairs."""
    from padra_b200.experts import bf16_values, zipf_routing

    host, table, k = make(1, hidden, inter, rate, 500 + hidden + tokens, gpu)
    ids, w = zipf_routing(tokens, seed=tokens, device=gpu)
    g = torch.Generator(device=gpu)
    g.manual_seed(tokens)
    dx = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    xa, xb = dx.clone(), dx.clone()
    ga, ua, da = (t.clone() for t in k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xa, tokens, tensor_memory=True))
    gb, ub, db = k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dx, xb, tokens, tensor_memory=False)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert_close_rows(bf16_bits_to_f32(u16(ga)), bf16_bits_to_f32(u16(gb)), "gate: tensor-memory vs small-tile kernel")
    assert_close_rows(bf16_bits_to_f32(u16(ua)), bf16_bits_to_f32(u16(ub)), "up: tensor-memory vs small-tile kernel")
    a, b = xa.cpu().numpy().astype(np.float64), xb.cpu().numpy().astype(np.float64)
    assert (np.linalg.norm(a - b, axis=1) <= 1e-2 * np.linalg.norm(b, axis=1)).all()
    floor = np.maximum(np.abs(b), np.sqrt((b ** 2).mean(axis=1, keepdims=True)))
    assert (np.abs(a - b) <= 3e-2 * floor).all()
    h_ids, h_x, gate = ids.cpu().numpy().reshape(-1), dx.cpu().numpy(), bf16_bits_to_f32(u16(ga))
    for pair in (0, tokens * 4 + 1, tokens * 8 - 1):
        data, suh, svh = host.get(0, int(h_ids[pair]), 0)
        want, bad = oracle.linear(oracle.matrix(data, suh, svh, inter, hidden, rate), h_x[pair // 8])
        assert not bad
        assert_close_rows(gate[pair][None], want[None], f"gate row of pair {pair} vs oracle")


def test_config3_full_shape_against_oracle(oracle, gpu):
    """The graded prefill configuration itself: 2048 tokens, hidden 2048 / intermediate 1024, K4, top-8 of 64 with
    Zipf(1.1) popularity.  The whole layer against the oracle for 72 pairs spread over the hottest expert, a middle one
    and the coldest one (gate, up, down rows of each pair, and the layer's output row of each pair's token through a
    combine over the kernel's own down rows), and gate/up/down against the small-tile kernel on every row."""
    from padra_b200.experts import ExpertKernels, ExpertTable, bf16_values, zipf_routing
    hidden, inter, tokens, rate = 2048, 1024, 2048, 4
    table = ExpertTable(1, hidden, inter, rate, gpu).fill_random(31)
    k = ExpertKernels(table)
    ids, w = zipf_routing(tokens, seed=4, device=gpu)
    g = torch.Generator(device=gpu)
    g.manual_seed(4)
    dn = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    dx = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    xa, xb = dx.clone(), dx.clone()
    ga, ua, da = (t.clone() for t in k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dn, xa, tokens, tensor_memory=True))
    gb, ub, db = k.prefill_layer(0, ids.reshape(-1), w.reshape(-1), dn, xb, tokens, tensor_memory=False)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert_close_rows(bf16_bits_to_f32(u16(ga)), bf16_bits_to_f32(u16(gb)), "gate: tensor-memory vs small-tile kernel")
    assert_close_rows(bf16_bits_to_f32(u16(ua)), bf16_bits_to_f32(u16(ub)), "up: tensor-memory vs small-tile kernel")
    a, b = bf16_bits_to_f32(u16(da)).astype(np.float64), bf16_bits_to_f32(u16(db)).astype(np.float64)
    assert (np.linalg.norm(a - b, axis=1) <= 1e-2 * np.linalg.norm(b, axis=1)).all()

    h_ids, h_n = ids.cpu().numpy().reshape(-1), dn.cpu().numpy()
    counts = np.bincount(h_ids, minlength=64)
    order = np.argsort(-counts)
    chosen = [int(order[0]), int(order[32]), int(order[-1] if counts[order[-1]] else order[np.nonzero(counts[order])[0][-1]])]
    assert counts[chosen[0]] > 1024 and counts[chosen[2]] < 128, counts  # the imbalance the configuration is about
    gate, up, down = bf16_bits_to_f32(u16(ga)), bf16_bits_to_f32(u16(ua)), bf16_bits_to_f32(u16(da))
    checked = 0
    for e in chosen:
        pairs = np.nonzero(h_ids == e)[0]
        m = [oracle.matrix(*table.host_matrix(0, e, part), *table.shape(part), rate) for part in range(3)]
        for pair in pairs[np.linspace(0, len(pairs) - 1, 24).astype(int)]:  # first, last and evenly between
            x_row = h_n[pair // 8]
            want_g, bad_g = oracle.linear(m[0], x_row)
            want_u, bad_u = oracle.linear(m[1], x_row)
            assert not bad_g and not bad_u
            assert_close_rows(gate[pair][None], want_g[None], f"gate row, expert {e}, pair {pair}")
            assert_close_rows(up[pair][None], want_u[None], f"up row, expert {e}, pair {pair}")
            act = oracle.swiglu(want_g, want_u)
            want_d, bad_d = oracle.linear(m[2], act)
            assert not bad_d
            assert_close_rows(down[pair][None], want_d[None], f"down row, expert {e}, pair {pair}", chained=True)
            checked += 1
    assert checked == 72
    # the combine over the kernel's own down rows, every token
    want_x, bad = oracle.combine(dx.cpu().numpy(), down.reshape(tokens, 8, hidden), w.cpu().numpy().reshape(tokens, 8))
    assert not bad
    assert np.array_equal(xa.cpu().numpy(), want_x), "combine over the down rows differs from the oracle's"


@pytest.mark.parametrize("rows_entry", [False, True])
def test_prefill_rejects_a_table_of_another_rate(gpu, rows_entry):
    """A descriptor table whose format does not match the requested rate: detected from the descriptor before anything
    is read through it, by the input transform as well as by the grouped GEMM; the flag is raised, nothing is written."""
    from padra_b200 import binding as B
    from padra_b200.experts import bf16_values, zipf_routing

    hidden, inter, tokens = 256, 128, 16
    _, table, k = make(1, hidden, inter, 4, 601, gpu)
    ids, w = zipf_routing(tokens, seed=1, device=gpu)
    ids = ids.reshape(-1)
    dx = bf16_values(torch.randn((tokens, hidden), device=gpu))
    sched = k.group_and_schedule(ids, tokens)
    groups, counts, tiles, tile_count = sched
    out = torch.full((tokens * 8, inter), 0x7777, dtype=torch.uint16, device=gpu)
    transformed = torch.zeros((tokens * 8, hidden), dtype=torch.float16, device=gpu)
    wrong_rate = 6
    if rows_entry:
        rows = bf16_values(torch.randn((tokens * 8, hidden), device=gpu)).to(torch.bfloat16).view(torch.uint16)
        st = k.lib.padra_exl3_prefill_rows_launch(table.descriptors.data_ptr(), 0, 0, B.ptr(groups), B.ptr(counts), tokens, tokens * 8,
                                                  B.ptr(rows), B.ptr(out), None, None, B.ptr(k.table), B.ptr(transformed), B.ptr(k.bad),
                                                  B.stream_handle(), wrong_rate, hidden, inter, 0, 0)
    else:
        st = k.lib.padra_exl3_prefill_launch(table.descriptors.data_ptr(), 0, 0, B.ptr(ids), B.ptr(groups), B.ptr(counts), B.ptr(tiles),
                                             B.ptr(tile_count), B.ptr(dx), B.ptr(out), None, None, B.ptr(k.table), B.ptr(transformed),
                                             tokens, B.ptr(k.bad), B.stream_handle(), None, 1, wrong_rate, hidden, inter)
    assert st == 0
    torch.cuda.synchronize()
    assert k.bad_flag() == 1
    assert int((u16(out) != 0x7777).sum()) == 0, "a refused projection wrote output rows"
    assert float(transformed.abs().max()) == 0.0, "a refused projection wrote transformed rows"
