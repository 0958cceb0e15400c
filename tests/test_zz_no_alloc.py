"""The decode layer on the library's built-in scratch array (padra_exl3_moe_decode_layer_static), through the C ABI.

Collected last on purpose: the entry point shares one device array between all calls of the process, so it has to give
the right answer after everything else has run as well as in a fresh process.  Its results are compared with the
caller-workspace entry point's on the same inputs, two calls in a row (the second call meets the first call's
left-overs in the array)."""
import numpy as np
import pytest
import torch

from tests.helpers import assert_close_rows
from tests.test_gpu_decode import make, routed_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens", [1, 4])
def test_static_scratch_layer_equals_workspace_layer_twice(oracle, gpu, tokens):
    hidden, inter = 512, 256
    _, _, k = make(2, hidden, inter, 4, 97, gpu)
    for call in range(2):
        x, ids, w = routed_inputs(oracle, tokens, hidden, 300 + call)
        normalized, _, _ = routed_inputs(oracle, tokens, hidden, 400 + call)
        dids = torch.from_numpy(ids.reshape(-1)).to(gpu)
        dw = torch.from_numpy(w.reshape(-1)).to(gpu)
        dn = torch.from_numpy(normalized).to(gpu)
        want, got = torch.from_numpy(x).to(gpu), torch.from_numpy(x).to(gpu)
        k.moe_decode_layer(call, dids, dw, dn, want, tokens)
        k.moe_decode_layer_static(call, dids, dw, dn, got, tokens)
        torch.cuda.synchronize()
        assert k.bad_flag() == 0
        assert_close_rows(got.cpu().numpy(), want.cpu().numpy(), f"static scratch vs workspace, call {call}", chained=True)
        assert not np.array_equal(got.cpu().numpy(), x), "the layer did not change the residual stream"


def test_static_scratch_refuses_what_does_not_fit(gpu):
    from padra_b200 import binding as B

    hidden, inter = 2048, 1024
    lib = B.load()
    needed = lib.padra_exl3_moe_decode_workspace_bytes(16, hidden, inter)
    assert needed > (4 << 20)
    _, _, k = make(1, 256, 128, 4, 5, gpu)
    dummy = torch.zeros(16 * hidden, device=gpu)
    ids = torch.zeros(16 * 8, dtype=torch.int32, device=gpu)
    st = lib.padra_exl3_moe_decode_layer_static(k.t.descriptors.data_ptr(), 0, ids.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                                dummy.data_ptr(), 16, 4, hidden, inter, k.table.data_ptr(), k.bad.data_ptr(), None)
    assert st == B.RESOURCE_EXHAUSTED
