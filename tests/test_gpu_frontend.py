"""GPU parity tests of the callers either side of the expert projections: exact-rank routing, the fused routing +
grouping + tile schedule of a prefill chunk, and the two RMS norms.  All integer results and all floating-point results
here are required to be equal bit for bit: the kernels keep the reference's operation order."""
import numpy as np
import pytest
import torch

from oracle import exl3_oracle as O
from tests.test_gpu_decode import make, needs_ref

pytestmark = pytest.mark.gpu


def bf16_logits(rng, tokens):
    return O.bf16_round(rng.standard_normal((tokens, 64)).astype(np.float32))


@pytest.mark.parametrize("tokens", [1, 5, 37, 2048])
def test_route_equals_oracle(oracle, gpu, tokens):
    _, _, k = make(1, 256, 128, 4, 801, gpu)
    rng = np.random.default_rng(tokens)
    logits = bf16_logits(rng, tokens)
    if tokens > 4:
        logits[1, :] = 0.5  # every expert tied: the lowest indices win
        logits[2, 10:30] = logits[2, 9]  # a run of ties across the top-8 boundary
        logits[3, :] = np.linspace(-80.0, 80.0, 64, dtype=np.float32)  # probabilities that underflow
    want_ids, want_w, bad = oracle.route(logits)
    assert not bad
    ids, w = k.route(torch.from_numpy(logits).to(gpu))
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert np.array_equal(ids.cpu().numpy(), want_ids)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), want_w.view(np.uint32)), "routing weights differ from the oracle's bits"
    assert (np.diff(ids.cpu().numpy(), axis=1) > 0).all()


def test_route_refuses_non_finite_logits(gpu):
    _, _, k = make(1, 256, 128, 4, 803, gpu)
    logits = torch.zeros((3, 64), device=gpu)
    logits[1, 7] = float("inf")
    ids, w = k.route(logits)
    torch.cuda.synchronize()
    assert k.bad_flag() == 1
    assert ids[1].abs().sum().item() == 0 and w[1].abs().sum().item() == 0.0
    assert (ids[0].cpu().numpy() == np.arange(8)).all()  # an all-equal row routed before the flag was seen, or zeroed
    k.reset_bad()


@needs_ref
def test_route_equals_reference_kernel(gpu):
    from padra_b200 import binding as B

    _, _, k = make(1, 256, 128, 4, 805, gpu)
    ref = O.RefKernels()
    logits = torch.from_numpy(bf16_logits(np.random.default_rng(11), 300)).to(gpu)
    ids, w = k.route(logits)
    rids, rw = torch.zeros_like(ids), torch.zeros_like(w)
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    ref.ref_route_rank_exact(B.ptr(logits), B.ptr(rids), B.ptr(rw), 300, B.ptr(bad), B.stream_handle())
    torch.cuda.synchronize()
    assert int(bad.item()) == 0 and k.bad_flag() == 0
    assert torch.equal(ids, rids) and torch.equal(w.view(torch.int32), rw.view(torch.int32))


@pytest.mark.parametrize("tokens", [4, 33, 257, 2048])
def test_route_group_schedule_in_one_launch(oracle, gpu, tokens):
    _, _, k = make(1, 256, 128, 4, 807, gpu)
    rng = np.random.default_rng(100 + tokens)
    logits = bf16_logits(rng, tokens)
    logits[:, :6] += 2.0  # popular experts: uneven groups, several tiles per expert
    d_logits = torch.from_numpy(logits).to(gpu)
    for call in range(2):  # the second call finds the ticket word as the first one left it
        ids, w, (groups, counts, tiles, tile_count) = k.route_group_schedule(d_logits)
        torch.cuda.synchronize()
        assert k.bad_flag() == 0
        want_ids, want_w, bad = oracle.route(logits)
        assert not bad
        assert np.array_equal(ids.cpu().numpy(), want_ids)
        assert np.array_equal(w.cpu().numpy().view(np.uint32), want_w.view(np.uint32))
        og, oc, bad = oracle.group(want_ids, tokens)
        assert not bad
        assert (counts.cpu().numpy() == oc).all()
        g, og = groups.cpu().numpy().reshape(64, tokens), og.reshape(64, tokens)
        for e in range(64):
            assert (g[e, : oc[e]] == og[e, : oc[e]]).all()
        ot, bad = oracle.schedule(oc, tokens)
        assert not bad
        n = int(tile_count.item())
        assert n == len(ot) and (tiles.cpu().numpy()[:n] == ot).all()
        # and the separate entry points agree
        groups2, counts2, tiles2, tile_count2 = k.group_and_schedule(ids.reshape(-1), tokens)
        assert torch.equal(counts, counts2) and torch.equal(tile_count, tile_count2) and torch.equal(tiles[:n], tiles2[:n])


def weight_bits(rng, hidden):
    return (O.bf16_round((1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)).view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("hidden,rows,with_residual", [(2048, 1, True), (2304, 5, True), (2048, 16, False), (128, 3, True)])
def test_residual_norm_equals_oracle(oracle, gpu, hidden, rows, with_residual):
    _, _, k = make(1, 256, 128, 4, 809, gpu)
    rng = np.random.default_rng(hidden + rows)
    x = O.bf16_round((3.0 * rng.standard_normal((rows, hidden))).astype(np.float32))
    residual = O.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32)) if with_residual else None
    wb = weight_bits(rng, hidden)
    want_x, want_n, want_s, bad = oracle.residual_norm(x, residual, wb)
    assert not bad
    dx = torch.from_numpy(x).to(gpu)
    dn = torch.zeros_like(dx)
    stats = torch.zeros((rows, 2), device=gpu)
    k.residual_norm(dx, None if residual is None else torch.from_numpy(residual).to(gpu), dn, torch.from_numpy(wb.view(np.int16)).to(gpu), stats)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert np.array_equal(dx.cpu().numpy().view(np.uint32), want_x.view(np.uint32))
    assert np.array_equal(stats.cpu().numpy().view(np.uint32), want_s.view(np.uint32)), "variance / inverse root differ"
    assert np.array_equal(dn.cpu().numpy().view(np.uint32), want_n.view(np.uint32))


@pytest.mark.parametrize("hidden,rows", [(2048, 1), (2304, 4)])
def test_combine_norm_equals_oracle_and_the_two_step_form(oracle, gpu, hidden, rows):
    _, _, k = make(1, hidden, 128, 4, 811, gpu)  # the combine wrapper takes the row length from its table
    rng = np.random.default_rng(hidden)
    x = O.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32))
    down = O.bf16_round((4.0 * rng.standard_normal((rows, 8, hidden))).astype(np.float32))
    routing = rng.random((rows, 8)).astype(np.float32) + 0.1
    routing = O.bf16_round(routing / routing.sum(axis=1, keepdims=True))
    wb = weight_bits(rng, hidden)
    want_x, want_n, want_s, bad = oracle.combine_norm(x, down, routing, wb)
    assert not bad
    dx, dd, dr = torch.from_numpy(x).to(gpu), torch.from_numpy(down).to(gpu), torch.from_numpy(routing).to(gpu)
    dw = torch.from_numpy(wb.view(np.int16)).to(gpu)
    fused_x, fused_n = dx.clone(), torch.zeros_like(dx)
    k.combine_norm(fused_x, dd, dr, fused_n, dw)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert np.array_equal(fused_x.cpu().numpy().view(np.uint32), want_x.view(np.uint32))
    assert np.array_equal(fused_n.cpu().numpy().view(np.uint32), want_n.view(np.uint32))
    # combine, then the norm without a residual: the same bits in two launches
    step_x, step_n = dx.clone(), torch.zeros_like(dx)
    k.combine(step_x, dd.reshape(rows * 8, hidden), dr.reshape(-1), rows)
    k.residual_norm(step_x, None, step_n, dw)
    torch.cuda.synchronize()
    assert torch.equal(step_x, fused_x) and torch.equal(step_n, fused_n)


@needs_ref
@pytest.mark.parametrize("rows", [1, 5])
def test_residual_norm_equals_reference_kernel(gpu, rows):
    """ResidualPostNormWideExact itself, compiled unmodified for this GPU, at its own shape (2304 elements)."""
    from padra_b200 import binding as B

    _, _, k = make(1, 256, 128, 4, 813, gpu)
    ref = O.RefKernels()
    hidden = 2304
    rng = np.random.default_rng(rows)
    x = torch.from_numpy(O.bf16_round((2.0 * rng.standard_normal((rows, hidden))).astype(np.float32))).to(gpu)
    residual = torch.from_numpy(O.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32))).to(gpu)
    dw = torch.from_numpy(weight_bits(rng, hidden).view(np.int16)).to(gpu)
    ours_x, ours_n, ours_s = x.clone(), torch.zeros_like(x), torch.zeros((rows, 2), device=gpu)
    ref_x, ref_n, ref_s = x.clone(), torch.zeros_like(x), torch.zeros((rows, 2), device=gpu)
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    k.residual_norm(ours_x, residual, ours_n, dw, ours_s)
    ref.ref_residual_post_norm(B.ptr(ref_x), B.ptr(residual), B.ptr(ref_n), B.ptr(dw), B.ptr(bad), B.ptr(ref_s), rows, B.stream_handle())
    torch.cuda.synchronize()
    assert int(bad.item()) == 0 and k.bad_flag() == 0
    assert torch.equal(ours_x, ref_x) and torch.equal(ours_s.view(torch.int32), ref_s.view(torch.int32)) and torch.equal(ours_n, ref_n)
