"""The C++ host above the C ABI (padra_b200/host): artifact -> device arena -> descriptor table -> one decode layer, on
the GPU, against the same layer through the ctypes caller; and the Python artifact loader's table against the table the
artifact was saved from."""
import json
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.test_gpu_decode import make, routed_inputs

pytestmark = pytest.mark.gpu
TOOL = Path(__file__).resolve().parent.parent / "padra_b200" / "host" / "padra_host_tool"


@pytest.mark.parametrize("rate,tokens", [(4, 1), (3, 5), (6, 16)])
def test_cpp_host_runs_the_layer_from_an_artifact(oracle, gpu, tmp_path, rate, tokens):
    from padra_b200.experts import ExpertKernels, ExpertTable

    assert TOOL.exists(), "padra_b200/host/padra_host_tool is built by `python -m padra_b200.build` beside the library"
    hidden, inter, layer = 512, 256, 1
    _, table, k = make(2, hidden, inter, rate, 700 + rate, gpu)
    table.save_artifact(tmp_path / "model")
    x, ids, w = routed_inputs(oracle, tokens, hidden, 40 + tokens)
    normalized, _, _ = routed_inputs(oracle, tokens, hidden, 80 + tokens)
    blob = struct.pack("<4i", layer, tokens, hidden, inter) + ids.astype("<i4").tobytes() + w.astype("<f4").tobytes() + \
        normalized.astype("<f4").tobytes() + x.astype("<f4").tobytes()
    (tmp_path / "inputs.bin").write_bytes(blob)
    out = subprocess.run([str(TOOL), "decode", str(tmp_path / "model"), str(tmp_path / "inputs.bin"), str(tmp_path / "output.bin")],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert json.loads(out.stdout) == {"tokens": tokens, "layer": layer, "bad": 0}
    raw = (tmp_path / "output.bin").read_bytes()
    got = np.frombuffer(raw[:-4], dtype="<f4").reshape(tokens, hidden)
    assert struct.unpack("<i", raw[-4:])[0] == 0
    # the same layer through the ctypes caller on the table the artifact was saved from ...
    dids, dw = torch.from_numpy(ids.reshape(-1)).to(gpu), torch.from_numpy(w.reshape(-1)).to(gpu)
    dn, want = torch.from_numpy(normalized).to(gpu), torch.from_numpy(x).to(gpu)
    k.moe_decode_layer(layer, dids, dw, dn, want, tokens)
    torch.cuda.synchronize()
    assert k.bad_flag() == 0
    assert np.array_equal(got, want.cpu().numpy()), "C++ host and ctypes caller disagree"
    # ... and on a table loaded back from the artifact by the Python reader
    loaded = ExpertTable.from_artifact(tmp_path / "model", gpu)
    assert (loaded.layers, loaded.hidden, loaded.inter, loaded.rate) == (2, hidden, inter, rate)
    again = torch.from_numpy(x).to(gpu)
    ExpertKernels(loaded).moe_decode_layer(layer, dids, dw, dn, again, tokens)
    torch.cuda.synchronize()
    assert torch.equal(again, want)
