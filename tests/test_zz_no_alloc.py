"""The decode layer on the library's built-in scratch array (padra_exl3_moe_decode_layer_static), through the C ABI.

Collected last on purpose: the entry point shares one device array between all calls of the process, so it has to give
the right answer after everything else has run as well as in a fresh process.  Its results are compared with the
caller-workspace entry point's on the same inputs, two calls in a row (the second call meets the first call's
left-overs in the array).  Both entry points run the same deterministic pipeline, so the results must be equal bit for
bit."""
import numpy as np
import pytest
import torch

from tests.test_gpu_decode import make, routed_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rate,tokens", [(4, 1), (4, 4), (3, 2), (6, 3)])
def test_static_scratch_layer_equals_workspace_layer_twice(oracle, gpu, rate, tokens):
    hidden, inter = 512, 256
    _, _, k = make(2, hidden, inter, rate, 97, gpu)
    k.decode_workspace(tokens)  # the workspace entry point's buffer exists before free memory is sampled
    for call in range(2):
        x, ids, w = routed_inputs(oracle, tokens, hidden, 300 + call)
        normalized, _, _ = routed_inputs(oracle, tokens, hidden, 400 + call)
        dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
        dw = torch.from_numpy(w.reshape(-1)).to(gpu)
        dn = torch.from_numpy(normalized).to(gpu)
        want, got = torch.from_numpy(x).to(gpu), torch.from_numpy(x).to(gpu)
        k.moe_decode_layer(call, dids, dw, dn, want, tokens)
        if call == 0:
            k.moe_decode_layer_static(call, dids, dw, dn, got, tokens)  # first call: set-up (address look-up) happens here
            got.copy_(torch.from_numpy(x).to(gpu))
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        k.moe_decode_layer_static(call, dids, dw, dn, got, tokens)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after == free_before, "the allocation-free entry point changed the device's free memory"
        assert k.bad_flag() == 0
        assert torch.equal(got, want), f"static scratch vs workspace, call {call}"
        assert not np.array_equal(got.cpu().numpy(), x), "the layer did not change the residual stream"


def test_static_scratch_size_limit(oracle, gpu):
    """The benchmark shape (hidden 2048 / intermediate 1024) fits the 4 MiB array at every batch up to sixteen tokens; at
    hidden 4096 / intermediate 2048 nine tokens fit and ten do not.  The largest batch that fits is run and compared,
    the first one that does not fit is refused without touching anything."""
    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable

    lib = B.load()
    limit = 4 << 20
    assert lib.padra_exl3_moe_decode_workspace_bytes(16, 2048, 1024) <= limit
    assert lib.padra_exl3_moe_decode_workspace_bytes(16, 2304, 896) <= limit
    hidden, inter = 4096, 2048
    assert lib.padra_exl3_moe_decode_workspace_bytes(9, hidden, inter) <= limit
    assert lib.padra_exl3_moe_decode_workspace_bytes(10, hidden, inter) > limit
    table = ExpertTable(1, hidden, inter, 4, gpu).fill_random(2)
    k = ExpertKernels(table)
    x, ids, w = routed_inputs(oracle, 10, hidden, 500)
    dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
    dw = torch.from_numpy(w.reshape(-1)).to(gpu)
    dx = torch.from_numpy(x).to(gpu)
    fits = dx[:9].contiguous()
    want, got = fits.clone(), fits.clone()
    k.moe_decode_layer(0, dids[:72], dw[:72], fits, want, 9)
    k.moe_decode_layer_static(0, dids[:72], dw[:72], fits, got, 9)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0 and torch.equal(got, want) and not torch.equal(got, fits)
    refused = dx.clone()
    st = lib.padra_exl3_moe_decode_layer_static(table.descriptors.data_ptr(), 0, dids.data_ptr(), dw.data_ptr(), dx.data_ptr(),
                                                refused.data_ptr(), 10, 4, hidden, inter, k.table.data_ptr(), k.bad.data_ptr(), None)
    assert st == B.RESOURCE_EXHAUSTED
    torch.cuda.synchronize()
    assert torch.equal(refused, dx), "a refused call must not touch the residual stream"
