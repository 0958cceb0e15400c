"""GPU parity tests of the decode-side entry points, called through the C ABI.

Integer work (trellis decode, unions) must be bit-exact against the CPU oracle; projections and whole layers
must be within the 1e-2 relative tolerance of the oracle (which restates the reference's FP32 arithmetic), and
-- where the reference's own kernels were compiled for this GPU (oracle/_ref) -- of those kernels too.
"""
import numpy as np
import pytest
import torch

from oracle import exl3_oracle as O
from tests.helpers import assert_close_rows, u16

pytestmark = pytest.mark.gpu
RATES = [3, 4, 6]


def make(layers, hidden, inter, rate, seed, gpu):
    from padra_b200.experts import ExpertKernels, ExpertTable

    host = O.HostMatrices(layers, hidden, inter, rate, seed=seed)
    table = ExpertTable(layers, hidden, inter, rate, gpu).fill_from_host(host)
    return host, table, ExpertKernels(table)


def routed_inputs(oracle, tokens, hidden, seed):
    rng = np.random.default_rng(seed)
    x = O.bf16_round(rng.standard_normal((tokens, hidden)).astype(np.float32))
    ids, w, bad = oracle.route(O.bf16_round(rng.standard_normal((tokens, 64)).astype(np.float32)))
    assert not bad
    return x, ids, w


CODEC_FORMS = [False, True]  # byte sums on the integer pipe (dp4a) / on the tensor cores (integer mma)


@pytest.mark.parametrize("tensor_form", CODEC_FORMS)
@pytest.mark.parametrize("rate", RATES)
def test_weight_decode_bit_exact(oracle, gpu, rate, tensor_form):
    host, table, k = make(1, 256, 128, rate, 11, gpu)
    for e in (0, 17, 63):
        for part in (0, 2):
            rows, cols = table.shape(part)
            got = u16(k.decode_weights(0, e, part, tensor_form=tensor_form))
            want = oracle.decode_matrix(host.get(0, e, part)[0], rows, cols, rate)
            assert (got == want).all(), (rate, e, part, int((got != want).sum()))
    assert k.bad_flag() == 0


@pytest.mark.parametrize("tensor_form", CODEC_FORMS)
@pytest.mark.parametrize("rate", RATES)
def test_weight_decode_bit_exact_full_size(oracle, gpu, rate, tensor_form):
    """One 1024 x 2048 matrix per rate: every one of its 2 Mi weights, through both forms of the codec."""
    from padra_b200.experts import ExpertKernels, ExpertTable

    table = ExpertTable(1, 2048, 1024, rate, gpu).fill_random(3)
    k = ExpertKernels(table)
    got = u16(k.decode_weights(0, 5, 0, tensor_form=tensor_form))
    want = oracle.decode_matrix(table.host_matrix(0, 5, 0)[0], 1024, 2048, rate)
    assert (got == want).all()
    assert k.bad_flag() == 0


@pytest.mark.parametrize("rate", RATES)
def test_single_token_projections_and_layer(oracle, gpu, rate):
    hidden, inter = 512, 256
    host, table, k = make(2, hidden, inter, rate, 21 + rate, gpu)
    x, ids, w = routed_inputs(oracle, 1, hidden, 5)
    want, bad, (cg, cu, ca, cd) = oracle.moe_layer(host.table, 1, ids, w, x, hidden, inter, capture=True)
    assert not bad
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    gate = torch.zeros((8, inter), device=gpu)
    up = torch.zeros((8, inter), device=gpu)
    down = torch.zeros((8, hidden), device=gpu)
    k.decode_launch(1, 0, dids, dx, gate, up)
    assert_close_rows(gate.cpu().numpy(), cg, "gate")
    assert_close_rows(up.cpu().numpy(), cu, "up")
    k.silu_activate(gate, up)
    assert_close_rows(gate.cpu().numpy(), ca, "activation")
    act = torch.from_numpy(ca).to(gpu)  # feed the oracle's activation so the down check stands alone
    k.decode_launch(1, 2, dids, act, down)
    assert_close_rows(down.cpu().numpy(), cd, "down")
    # the small-batch launcher gives the same rows, one part per call
    single = torch.zeros((8, inter), device=gpu)
    k.expert_launch(1, 1, dids, dx, single, 1)
    assert torch.equal(single, up)
    # whole layer in one call
    xs = dx.clone()
    k.moe_decode_layer(1, dids, torch.from_numpy(w.reshape(-1)).to(gpu), dx, xs, 1)
    assert_close_rows(xs.cpu().numpy(), want, "layer", chained=True)
    assert k.bad_flag() == 0


@pytest.mark.parametrize("rate", RATES)
@pytest.mark.parametrize("tokens", [2, 5, 16])
def test_multi_token_layer(oracle, gpu, rate, tokens):
    hidden, inter = 256, 128
    host, table, k = make(1, hidden, inter, rate, 31, gpu)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 6 + tokens)
    want, bad = oracle.moe_layer(host.table, 0, ids, w, x, hidden, inter)
    assert not bad
    dx = torch.from_numpy(x).to(gpu)
    xs = dx.clone()
    k.moe_decode_layer(0, torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu), dx, xs, tokens)
    assert_close_rows(xs.cpu().numpy(), want, f"layer M={tokens}", chained=True)
    assert k.bad_flag() == 0


FORMS = ["moe_decode_layer"]


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("rate", RATES)
@pytest.mark.parametrize("tokens", [1, 3, 8, 13])
def test_layer_call_matches_separate_launches(oracle, gpu, rate, tokens, form):
    """The whole-layer call (two launches, epilogues inside) against the per-part entry points launched one after
    another."""
    hidden, inter = 512, 384
    host, table, k = make(1, hidden, inter, rate, 97, gpu)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 40 + tokens)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dw = torch.from_numpy(w.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    fused, separate = dx.clone(), dx.clone()
    getattr(k, form)(0, dids, dw, dx, fused, tokens)
    k.moe_decode_layer_unfused(0, dids, dw, dx, separate, tokens)
    assert_close_rows(fused.cpu().numpy(), separate.cpu().numpy(), "layer call vs separate launches", chained=True)
    again = dx.clone()
    getattr(k, form)(0, dids, dw, dx, again, tokens)  # the workspace was left clean: a second call gives the same bits
    assert torch.equal(again, fused)
    assert k.bad_flag() == 0


@pytest.mark.parametrize("form", FORMS)
def test_layer_call_mellum_dims(oracle, gpu, form):
    """Hidden 2304 / intermediate 896 (18 and 7 blocks of 128): non-power-of-two chunk and slice bookkeeping."""
    from padra_b200.experts import ExpertKernels, ExpertTable

    hidden, inter = 2304, 896
    tokens = 5
    table = ExpertTable(1, hidden, inter, 4, gpu).fill_random(9)
    k = ExpertKernels(table)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 50)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dw = torch.from_numpy(w.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    fused, separate = dx.clone(), dx.clone()
    getattr(k, form)(0, dids, dw, dx, fused, tokens)
    k.moe_decode_layer_unfused(0, dids, dw, dx, separate, tokens)
    assert_close_rows(fused.cpu().numpy(), separate.cpu().numpy(), "fused vs separate launches, 2304/896", chained=True)
    assert k.bad_flag() == 0


@pytest.mark.parametrize("form", FORMS)
def test_layer_call_rejects_bad_ids_and_descriptors(gpu, form):
    _, table, k = make(1, 256, 128, 4, 101, gpu)
    x = torch.ones((1, 256), device=gpu)
    w = torch.full((8,), 0.125, device=gpu)
    out = x.clone()
    getattr(k, form)(0, torch.tensor([0, 1, 2, 64, 4, 5, 6, 7], dtype=torch.int32, device=gpu), w, x, out, 1)
    torch.cuda.synchronize()
    assert k.bad_flag() == 1 and torch.equal(out, x)  # refused before any work
    k.reset_bad()
    # a table of another rate: every chunk's descriptor check fails, the step completes and is flagged
    from padra_b200 import binding as B
    ws = k.decode_workspace(1)
    entry = getattr(k.lib, "padra_exl3_" + form)
    st = entry(table.descriptors.data_ptr(), 0, B.ptr(torch.arange(8, dtype=torch.int32, device=gpu)),
               B.ptr(w), B.ptr(x), B.ptr(out), 1, 6, 256, 128, B.ptr(k.table), B.ptr(ws), ws.numel(), B.ptr(k.bad), B.stream_handle())
    assert st == 0
    torch.cuda.synchronize()
    assert k.bad_flag() == 1
    k.reset_bad()
    good = x.clone()
    getattr(k, form)(0, torch.arange(8, dtype=torch.int32, device=gpu), w, x, good, 1)  # and the workspace is reusable
    torch.cuda.synchronize()
    assert k.bad_flag() == 0 and not torch.equal(good, x)


@pytest.mark.parametrize("form", FORMS)
def test_layer_call_repeated_many_times_single_token(oracle, gpu, form):
    """Forty back-to-back single-token steps over two layers of the benchmark shape: every one must agree with the
    per-part launches and leave the error flag down (guards the ticket counters that hand the epilogues out)."""
    from padra_b200.experts import ExpertKernels, ExpertTable, bf16_values, route_topk

    hidden, inter = 2048, 1024
    table = ExpertTable(2, hidden, inter, 4, gpu).fill_random(5)
    k = ExpertKernels(table)
    g = torch.Generator(device=gpu)
    g.manual_seed(77)
    for it in range(40):
        ids, w = route_topk(bf16_values(torch.randn((1, 64), device=gpu, generator=g)))
        n = bf16_values(torch.randn((1, hidden), device=gpu, generator=g))
        x = bf16_values(torch.randn((1, hidden), device=gpu, generator=g))
        a, b = x.clone(), x.clone()
        getattr(k, form)(it % 2, ids.reshape(-1), w.reshape(-1), n, a, 1)
        k.moe_decode_layer_unfused(it % 2, ids.reshape(-1), w.reshape(-1), n, b, 1)
        assert_close_rows(a.cpu().numpy(), b.cpu().numpy(), f"step {it}", chained=True)
    assert k.bad_flag() == 0


def host_experts(table, layer, experts):
    """Oracle-side descriptor table holding host copies of just the given experts of one layer."""
    mats = (O.Matrix * (64 * 3))()
    keep = []
    for e in sorted(set(int(e) for e in experts)):
        for part in range(3):
            data, suh, svh = table.host_matrix(layer, e, part)
            keep.append((data, suh, svh))
            m = mats[e * 3 + part]
            m.data, m.suh, m.svh = data.ctypes.data, suh.ctypes.data, svh.ctypes.data
            m.rows, m.cols = table.shape(part)
            m.format = O.FORMAT_OF_RATE[table.rate]
    return mats, keep


@pytest.mark.parametrize("rate", RATES)
@pytest.mark.parametrize("tokens", [1, 2, 5, 16])
def test_graded_shape_layer_against_oracle(oracle, gpu, rate, tokens):
    """The benchmark's decode shape (64 experts, hidden 2048, intermediate 1024) at every rate and batch of the rate and
    batch sweep, routing drawn per token from seeded logits: the whole-layer call against the oracle.  Sixteen tokens
    take the 16-row form of the kernels and touch most of the 64 experts."""
    hidden, inter = 2048, 1024
    from padra_b200.experts import ExpertKernels, ExpertTable

    table = ExpertTable(1, hidden, inter, rate, gpu).fill_random(rate)
    k = ExpertKernels(table)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 100 * rate + tokens)
    normalized, _, _ = routed_inputs(oracle, tokens, hidden, 200 * rate + tokens)
    mats, keep = host_experts(table, 0, ids.reshape(-1))
    # the oracle's layer takes one activation for both roles; here the residual stream and the normalised input differ,
    # as they do in the model: out = x + (layer(normalized) - normalized)
    want_n, bad = oracle.moe_layer(mats, 0, ids, w, normalized, hidden, inter)
    assert not bad
    dn = torch.from_numpy(normalized).to(gpu)
    got_n = dn.clone()
    dids, dw = torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu)
    k.moe_decode_layer(0, dids, dw, dn, got_n, tokens)
    assert_close_rows(got_n.cpu().numpy(), want_n, f"K{rate} M={tokens} layer at 2048/1024", chained=True)
    # and with a residual stream of its own: against the per-part entry points' chain on the same inputs
    dx = torch.from_numpy(x).to(gpu)
    fused, separate = dx.clone(), dx.clone()
    k.moe_decode_layer(0, dids, dw, dn, fused, tokens)
    k.moe_decode_layer_unfused(0, dids, dw, dn, separate, tokens)
    assert_close_rows(fused.cpu().numpy(), separate.cpu().numpy(), "layer call vs separate launches", chained=True)
    assert k.bad_flag() == 0


@pytest.mark.parametrize("rate", RATES)
def test_rows_sharing_an_expert_equal_single_row_results(gpu, rate):
    """The reference's own operator probe (tests/cuda/mtp_operators.cu:143-206): for 2..5 rows and eight route
    patterns, the row-union kernel must equal the M=1 kernel row by row, bit for bit."""
    hidden, inter = 256, 128
    _, table, k = make(1, hidden, inter, rate, 41, gpu)
    rng = np.random.default_rng(27)
    bits = (0x3D00 + rng.integers(0, 1024, size=5 * 8 * hidden)).astype(np.uint32) << 16
    x = bits.view(np.float32) * rng.choice([-1.0, 1.0], size=bits.size).astype(np.float32)
    dx = torch.from_numpy(x).to(gpu)
    cases = 0
    for rows in range(2, 6):
        for route in range(8):
            sel = np.array([[(route * 8 + s + (route % 3) * r * 8) % 64 for s in range(8)] for r in range(rows)], dtype=np.int32)
            dids = torch.from_numpy(sel.reshape(-1)).to(gpu)
            union = k.build_union(dids, rows)
            for part in (0, 2):
                width = hidden if part == 2 else inter
                cols = inter if part == 2 else hidden
                out = torch.zeros((rows * 8, width), device=gpu)
                out_up = torch.zeros((rows * 8, width), device=gpu)
                k.mtp_launch(0, part, union, rows, dx, out, out_up if part == 0 else None)
                ref = torch.zeros_like(out)
                ref_up = torch.zeros_like(out)
                for r in range(rows):
                    # M=1 launcher: gate/up read row pair/8 of its input, down reads row pair
                    xin = dx[r * cols:] if part == 0 else dx[r * 8 * cols:]
                    k.decode_launch(0, part, dids[r * 8:(r + 1) * 8], xin, ref[r * 8:(r + 1) * 8],
                                    ref_up[r * 8:(r + 1) * 8] if part == 0 else None)
                assert torch.equal(out, ref), (rows, route, part)
                if part == 0:
                    assert torch.equal(out_up, ref_up), (rows, route, "up")
                cases += 1
    assert cases == 64 and k.bad_flag() == 0


def test_union_tables_match_definition(gpu):
    _, table, k = make(1, 256, 128, 4, 43, gpu)
    rng = np.random.default_rng(9)
    for rows in (1, 3, 16):
        ids = np.stack([np.sort(rng.choice(64, 8, replace=False)) for _ in range(rows)]).astype(np.int32)
        masks, slots, active, count = (t.cpu().numpy() for t in k.build_union(torch.from_numpy(ids.reshape(-1)).to(gpu), rows))
        used = sorted(set(ids.reshape(-1).tolist()))
        assert int(count[0]) == len(used) and active[:len(used)].tolist() == used
        for e in range(64):
            want_mask = sum(1 << r for r in range(rows) if e in ids[r])
            assert int(masks[e]) & 0xFFFFFFFF == want_mask
            for r in range(rows):
                want = int(np.where(ids[r] == e)[0][0]) if e in ids[r] else -1
                assert slots[e, r] == want
    assert k.bad_flag() == 0


def test_bad_expert_id_sets_flag_without_fault(gpu):
    _, table, k = make(1, 256, 128, 4, 47, gpu)
    ids = torch.tensor([0, 1, 2, 99, 4, 5, 6, 7], dtype=torch.int32, device=gpu)
    x = torch.ones((1, 256), device=gpu)
    gate = torch.zeros((8, 128), device=gpu)
    up = torch.zeros((8, 128), device=gpu)
    k.decode_launch(0, 0, ids, x, gate, up)
    torch.cuda.synchronize()
    assert k.bad_flag() == 1
    # once raised, later launches leave their outputs alone
    gate.fill_(-7.0)
    k.decode_launch(0, 0, torch.arange(8, dtype=torch.int32, device=gpu), x, gate, up)
    torch.cuda.synchronize()
    assert float(gate.min()) == -7.0 and float(gate.max()) == -7.0
    k.reset_bad()
    # wrong rate for the table's format is a descriptor mismatch
    from padra_b200 import binding as B
    st = k.lib.padra_exl3_decode_launch(table.descriptors.data_ptr(), 0, 0, B.ptr(ids), B.ptr(x), B.ptr(gate), None, 8,
                                        B.ptr(k.bad), B.stream_handle(), None, B.ptr(up), 6, 256, 128)
    assert st == 0
    torch.cuda.synchronize()
    assert k.bad_flag() == 1


def test_overflowing_activation_sets_flag(gpu):
    _, table, k = make(1, 256, 128, 4, 53, gpu)
    x = torch.full((1, 256), 3.0e38, device=gpu).to(torch.bfloat16).float()
    gate = torch.zeros((8, 128), device=gpu)
    up = torch.zeros((8, 128), device=gpu)
    k.decode_launch(0, 0, torch.arange(8, dtype=torch.int32, device=gpu), x, gate, up)
    torch.cuda.synchronize()
    assert k.bad_flag() == 1


@pytest.mark.parametrize("form", FORMS)
def test_layer_call_is_graph_capturable_and_deterministic(oracle, gpu, form):
    hidden, inter = 512, 256
    tokens = 5
    _, table, k = make(1, hidden, inter, 4, 59, gpu)
    x, ids, w = routed_inputs(oracle, tokens, hidden, 8)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dw = torch.from_numpy(w.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    k.decode_workspace(tokens)
    eager = dx.clone()
    getattr(k, form)(0, dids, dw, dx, eager, tokens)
    static = dx.clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            getattr(k, form)(0, dids, dw, dx, static, tokens, stream=stream)
    results = []
    for _ in range(3):
        static.copy_(dx)
        graph.replay()
        torch.cuda.synchronize()
        results.append(static.clone())
    assert torch.equal(results[0], results[1]) and torch.equal(results[1], results[2])
    assert torch.equal(results[0], eager)
    assert k.bad_flag() == 0


# ---- against the reference's own kernels on this GPU ------------------------------------------------------
needs_ref = pytest.mark.skipif(not O.RefKernels.available(), reason="reference kernels not built (oracle/_ref)")


@needs_ref
@pytest.mark.parametrize("rate", RATES)
def test_against_reference_decode_kernels_mellum_dims(oracle, gpu, rate):
    """Mellum dimensions (hidden 2304, intermediate 896), the only shape the reference launchers accept:
    exl3_mma_dual::Launch, exl3_silu_lut::Activate, Combine vs this library, same inputs."""
    from padra_b200 import binding as B

    hidden, inter = 2304, 896
    from padra_b200.experts import ExpertKernels, ExpertTable

    table = ExpertTable(1, hidden, inter, rate, gpu).fill_random(100 + rate)
    k = ExpertKernels(table)
    ref = O.RefKernels()
    x, ids, w = routed_inputs(oracle, 1, hidden, 12)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dw = torch.from_numpy(w.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    s = B.stream_handle()
    D = table.descriptors.data_ptr()
    rg, ru = torch.zeros((8, inter), device=gpu), torch.zeros((8, inter), device=gpu)
    rd = torch.zeros((8, hidden), device=gpu)
    ref.ref_decode_dual_launch(D, 0, 0, B.ptr(dids), B.ptr(dx), B.ptr(rg), B.ptr(ru), 8, B.ptr(bad), s, rate)
    gate, up = torch.zeros_like(rg), torch.zeros_like(ru)
    k.decode_launch(0, 0, dids, dx, gate, up)
    assert_close_rows(gate.cpu().numpy(), rg.cpu().numpy(), "gate vs reference kernel")
    assert_close_rows(up.cpu().numpy(), ru.cpu().numpy(), "up vs reference kernel")
    rtable = torch.zeros(65536, dtype=torch.int16, device=gpu)
    ref.ref_silu_build(B.ptr(rtable), s)
    assert torch.equal(rtable, k.table.view(torch.int16)), "SwiGLU table differs from the reference's"
    assert (u16(k.table) == oracle.silu_table()).all(), "SwiGLU table differs from the oracle's"
    ref.ref_silu_activate(B.ptr(rg), B.ptr(ru), B.ptr(rtable), 8 * inter, B.ptr(bad), s)
    ours_act = rg.clone()  # same activation into both down projections
    ref.ref_decode_dual_launch(D, 0, 2, B.ptr(dids), B.ptr(rg), B.ptr(rd), None, 8, B.ptr(bad), s, rate)
    down = torch.zeros_like(rd)
    k.decode_launch(0, 2, dids, ours_act, down)
    assert_close_rows(down.cpu().numpy(), rd.cpu().numpy(), "down vs reference kernel")
    rx = dx.clone()
    ref.ref_combine(B.ptr(rx), B.ptr(rd), B.ptr(dw), 1, B.ptr(bad), s)
    ox = dx.clone()
    k.combine(ox, rd, dw, 1)
    assert torch.equal(ox, rx), "combine differs from the reference kernel on identical inputs"
    full = dx.clone()
    k.moe_decode_layer(0, dids, dw, dx, full, 1)
    assert_close_rows(full.cpu().numpy(), rx.cpu().numpy(), "layer vs reference kernels", chained=True)
    assert int(bad.item()) == 0 and k.bad_flag() == 0


@needs_ref
@pytest.mark.parametrize("rate", RATES)
def test_oracle_equals_reference_scalar_kernels(oracle, gpu, rate):
    """The reference's scalar path (InputHad, Dot, OutputHad: src/cuda/expert_exl3.cuh:32-113) run on this GPU
    against the C oracle: same operation order, so the outputs are expected to be identical bit for bit."""
    from padra_b200 import binding as B

    hidden, inter = 512, 256
    host, table, k = make(1, hidden, inter, rate, 61, gpu)
    ref = O.RefKernels()
    x, ids, w = routed_inputs(oracle, 1, hidden, 13)
    want, bad_o, (cg, cu, ca, cd) = oracle.moe_layer(host.table, 0, ids, w, x, hidden, inter, capture=True)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    out = torch.zeros((8, inter), device=gpu)
    s_in = torch.zeros((8, hidden), device=gpu)
    s_out = torch.zeros((8, hidden), device=gpu)
    ref.ref_simt_linear(table.descriptors.data_ptr(), 0, 0, B.ptr(dids), B.ptr(dx), B.ptr(out), B.ptr(s_in), B.ptr(s_out), 8,
                        B.ptr(bad), B.stream_handle(), inter, hidden)
    torch.cuda.synchronize()
    assert int(bad.item()) == 0
    got = out.cpu().numpy()
    mismatch = int((got.view(np.uint32) != cg.view(np.uint32)).sum())
    assert mismatch == 0, f"oracle vs reference scalar kernels: {mismatch} of {got.size} values differ"
    # and the reference's tensor-core decode kernel stays within tolerance of its own scalar path
    rg, ru = torch.zeros((8, inter), device=gpu), torch.zeros((8, inter), device=gpu)
    ref.ref_decode_dual(table.descriptors.data_ptr(), 0, 0, B.ptr(dids), B.ptr(dx), B.ptr(rg), B.ptr(ru), 8, B.ptr(bad),
                        B.stream_handle(), rate, inter)
    assert_close_rows(rg.cpu().numpy(), cg, "reference mma kernel vs oracle")


@needs_ref
def test_reference_row_union_kernel_agrees(oracle, gpu):
    """mtp_experts::Projection (reference) vs this library's union projection at M = 5."""
    from padra_b200 import binding as B

    hidden, inter, rate, rows = 512, 256, 4, 5
    host, table, k = make(1, hidden, inter, rate, 67, gpu)
    ref = O.RefKernels()
    x, ids, w = routed_inputs(oracle, rows, hidden, 14)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    masks = torch.zeros(64, dtype=torch.int32, device=gpu)
    slots = torch.zeros(64 * 5, dtype=torch.int32, device=gpu)
    active = torch.zeros(64, dtype=torch.int32, device=gpu)
    count = torch.zeros(1, dtype=torch.int32, device=gpu)
    s = B.stream_handle()
    ref.ref_mtp_build_union(B.ptr(dids), B.ptr(masks), B.ptr(slots), rows, B.ptr(bad), B.ptr(active), B.ptr(count), s)
    ours = k.build_union(dids, rows, slot_stride=5)
    assert torch.equal(ours[0], masks) and torch.equal(ours[1].reshape(-1), slots)
    assert torch.equal(ours[3], count) and torch.equal(ours[2][: int(count.item())], active[: int(count.item())])
    rg, ru = torch.zeros((rows * 8, inter), device=gpu), torch.zeros((rows * 8, inter), device=gpu)
    ref.ref_mtp_projection(table.descriptors.data_ptr(), 0, 0, B.ptr(masks), B.ptr(slots), rows, B.ptr(dx), B.ptr(rg), B.ptr(ru),
                           B.ptr(bad), s, B.ptr(active), B.ptr(count), rate, inter)
    gate, up = torch.zeros_like(rg), torch.zeros_like(ru)
    k.mtp_launch(0, 0, ours, rows, dx, gate, up, slot_stride=5)
    assert_close_rows(gate.cpu().numpy(), rg.cpu().numpy(), "union gate vs reference")
    assert_close_rows(up.cpu().numpy(), ru.cpu().numpy(), "union up vs reference")
    assert int(bad.item()) == 0 and k.bad_flag() == 0


@needs_ref
def test_mtp_draft_expert_layer_against_reference_sequence(oracle, gpu):
    """The expert layer of the MTP draft model (src/cuda/mtp.cuh:364-387): the reference's own sequence -- Route, the
    gate+up projection kernel, the table-free Activate, the down projection kernel, Combine -- on a one-layer K4 table of
    its own at the reference's dimensions, against one call of the whole-layer entry point (what the DraftExpertLayer
    forwarder issues).  Routing must be equal bit for bit, the layer within the chained tolerance."""
    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable

    hidden, inter, rate = 2304, 896, 4
    table = ExpertTable(1, hidden, inter, rate, gpu).fill_random(321)  # the draft model's own table: layer 0 only
    k = ExpertKernels(table)
    ref = O.RefKernels()
    rng = np.random.default_rng(17)
    logits = torch.from_numpy(O.bf16_round(rng.standard_normal((1, 64)).astype(np.float32))).to(gpu)
    normalized = torch.from_numpy(O.bf16_round(rng.standard_normal((1, hidden)).astype(np.float32))).to(gpu)
    x = torch.from_numpy(O.bf16_round(rng.standard_normal((1, hidden)).astype(np.float32))).to(gpu)
    s, D = B.stream_handle(), table.descriptors.data_ptr()
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    ids = torch.zeros(8, dtype=torch.int32, device=gpu)
    weights = torch.zeros(8, device=gpu)
    ref.ref_route(B.ptr(logits), B.ptr(ids), B.ptr(weights), 1, B.ptr(bad), s)
    ours_ids, ours_w = k.route(logits)
    assert torch.equal(ours_ids.reshape(-1), ids) and torch.equal(ours_w.reshape(-1).view(torch.int32), weights.view(torch.int32))
    gate, up = torch.zeros((8, inter), device=gpu), torch.zeros((8, inter), device=gpu)
    down = torch.zeros((8, hidden), device=gpu)
    want = x.clone()
    ref.ref_decode_dual_launch(D, 0, 0, B.ptr(ids), B.ptr(normalized), B.ptr(gate), B.ptr(up), 8, B.ptr(bad), s, rate)
    ref.ref_activate(B.ptr(gate), B.ptr(up), 1, s)
    ref.ref_decode_dual_launch(D, 0, 2, B.ptr(ids), B.ptr(gate), B.ptr(down), None, 8, B.ptr(bad), s, rate)
    ref.ref_combine(B.ptr(want), B.ptr(down), B.ptr(weights), 1, B.ptr(bad), s)
    got = x.clone()
    k.moe_decode_layer(0, ids, weights, normalized, got, 1)
    torch.cuda.synchronize()
    assert int(bad.item()) == 0 and k.bad_flag() == 0
    assert_close_rows(got.cpu().numpy(), want.cpu().numpy(), "draft expert layer vs the reference's sequence", chained=True)
