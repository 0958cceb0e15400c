"""The EXL3 artifact format (manifest.json + weights.bin): Python writer and reader, the C++ reader of the host tool, and
the forwarders header, all without a GPU."""
import json
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import exl3_oracle as O
from padra_b200 import artifact as A

ROOT = Path(__file__).resolve().parent.parent
TOOL = ROOT / "padra_b200" / "host" / "padra_host_tool"


def small_artifact(directory, rate=4, layers=1, hidden=256, inter=128, seed=3):
    rng = np.random.default_rng(seed)
    tensors = []
    for layer in range(layers):
        for e in range(64):
            for part in range(3):
                rows, cols = (hidden, inter) if part == 2 else (inter, hidden)
                data, suh, svh = O.synthetic_matrix(rng, rows, cols, rate)
                tensors.append((A.expert_tensor_name(layer, e, part), rows, cols, data, suh, svh))
    A.write(directory, rate, tensors)
    return tensors


@pytest.fixture(scope="module")
def host_tool():
    from padra_b200 import build

    build.build()
    assert TOOL.exists()
    return TOOL


@pytest.mark.parametrize("rate", [3, 4, 6])
def test_round_trip_and_layout(tmp_path, rate):
    tensors = small_artifact(tmp_path, rate=rate)
    art = A.load(tmp_path)
    assert art.rate == rate and art.layers == 1 and len(art.tensors) == 64 * 3
    payload = art.payload()
    for name, rows, cols, data, suh, svh in tensors[:7] + tensors[-5:]:
        t = art.tensors[name]
        assert (t.rows, t.cols) == (rows, cols)
        for (off, n), want in ((t.packed, data), (t.suh, suh), (t.svh, svh)):
            assert off % 256 == 0 and np.array_equal(payload[off:off + n], np.ascontiguousarray(want).view(np.uint8).reshape(-1))
    manifest = json.loads((tmp_path / "manifest.json").read_text())
    entry = manifest["tensors"][A.expert_tensor_name(0, 5, 2)]
    assert entry["codebook"] == "mul1" and entry["hadamard_block"] == 128 and entry["format"] == f"EXL3_K{rate}"
    assert manifest["profile"] == f"mellum16-exl3-k{rate}-fp8-bf16-v1"


def test_cpp_reader_accepts_what_python_writes(tmp_path, host_tool):
    small_artifact(tmp_path, layers=2)
    out = subprocess.run([str(host_tool), "check", str(tmp_path)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    summary = json.loads(out.stdout)
    art = A.load(tmp_path)
    assert summary == {"profile": art.profile, "rate": 4, "layers": 2, "tensors": 384, "weights_bytes": art.weights_bytes,
                       "weights_sha256": art.weights_sha256}


def corrupt(tmp_path, edit):
    path = tmp_path / "manifest.json"
    manifest = json.loads(path.read_text())
    edit(manifest)
    path.write_text(json.dumps(manifest))


def first(manifest):
    return manifest["tensors"][A.expert_tensor_name(0, 0, 0)]


CASES = {
    "misaligned region": (lambda m: first(m)["regions"]["suh"].__setitem__("offset", first(m)["regions"]["suh"]["offset"] + 2),
                          "invalid region range/alignment/bytes"),
    "wrong region size": (lambda m: first(m)["regions"]["packed"].__setitem__("bytes", 17), "invalid region range/alignment/bytes"),
    "other codebook": (lambda m: first(m).__setitem__("codebook", "3inst"), "unsupported EXL3 codec/transform"),
    "other hadamard block": (lambda m: first(m).__setitem__("hadamard_block", 64), "unsupported EXL3 codec/transform"),
    "rate mismatch": (lambda m: first(m).__setitem__("format", "EXL3_K6"), "tensor precision does not match selected hybrid"),
    "bad hash": (lambda m: m.__setitem__("weights_sha256", "0" * 64), "weight SHA-256 mismatch"),
    "payload size": (lambda m: m.__setitem__("weights_bytes", m["weights_bytes"] + 256), "truncated or oversized weight payload"),
    "schema": (lambda m: m.__setitem__("schema_version", 2), "unsupported manifest schema"),
    "weights path": (lambda m: m.__setitem__("weights_file", "../weights.bin"), "unsafe weights path"),
    "missing tensor region": (lambda m: first(m)["regions"].pop("svh"), "unknown/missing weight regions"),
}


@pytest.mark.parametrize("case", sorted(CASES))
def test_both_readers_reject_malformed_manifests(tmp_path, host_tool, case):
    small_artifact(tmp_path)
    edit, message = CASES[case]
    corrupt(tmp_path, edit)
    with pytest.raises(A.ArtifactError, match=message):
        A.load(tmp_path)
    out = subprocess.run([str(host_tool), "check", str(tmp_path)], capture_output=True, text=True)
    assert out.returncode == 1 and message in out.stderr, out.stderr


def test_both_readers_reject_a_zero_sidecar_and_overlapping_regions(tmp_path, host_tool):
    import hashlib

    small_artifact(tmp_path)
    art = A.load(tmp_path)
    payload = art.payload().copy()
    off, _ = art.tensors[A.expert_tensor_name(0, 3, 1)].svh
    payload[off + 10:off + 12] = 0  # one zero FP16 sidecar value
    (tmp_path / "weights.bin").write_bytes(payload.tobytes())
    corrupt(tmp_path, lambda m: m.__setitem__("weights_sha256", hashlib.sha256(payload.tobytes()).hexdigest()))
    for reader_error in ("zero EXL3 sidecar",):
        with pytest.raises(A.ArtifactError, match=reader_error):
            A.load(tmp_path)
        out = subprocess.run([str(host_tool), "check", str(tmp_path)], capture_output=True, text=True)
        assert out.returncode == 1 and reader_error in out.stderr
    # two tensors claiming the same bytes
    small_artifact(tmp_path)
    def overlap(m):
        m["tensors"][A.expert_tensor_name(0, 1, 0)]["regions"] = dict(first(m)["regions"])
    corrupt(tmp_path, overlap)
    with pytest.raises(A.ArtifactError, match="overlapping/noncanonical weight regions"):
        A.load(tmp_path, verify_payload=False)
    out = subprocess.run([str(host_tool), "check", str(tmp_path)], capture_output=True, text=True)
    assert out.returncode == 1 and "overlapping/noncanonical weight regions" in out.stderr


def test_sha256_of_the_cpp_reader_matches_hashlib(tmp_path, host_tool):
    """Payload sizes around the padding boundaries of SHA-256 (55, 56, 63, 64 bytes modulo 64)."""
    rng = np.random.default_rng(0)
    for extra_cols in (128, 256):  # different payload lengths
        tensors = []
        for e in range(64):
            for part in range(3):
                rows, cols = (128 + extra_cols, 128) if part == 2 else (128, 128 + extra_cols)
                tensors.append((A.expert_tensor_name(0, e, part), rows, cols, *O.synthetic_matrix(rng, rows, cols, 3)))
        A.write(tmp_path, 3, tensors)
        out = subprocess.run([str(host_tool), "check", str(tmp_path)], capture_output=True, text=True)
        assert out.returncode == 0, out.stderr  # the check compares its own SHA-256 with the manifest's (hashlib's)


def test_forwarders_header_compiles(tmp_path):
    """padra_b200/host/bind.hpp against the reference's own DeviceMatrix and Tile declarations when the reference checkout
    is present (PADRA_REFERENCE, else a directory `reference` beside the repository), else against the layout-identical stand-ins; every forwarder
    is instantiated."""
    reference = Path(os.environ.get("PADRA_REFERENCE", str(Path(__file__).resolve().parents[2] / "reference")))
    tile_header = reference / "src" / "runtime" / "exl3_masked_schedule.h"
    source = tmp_path / "forwarders.cpp"
    if tile_header.exists():
        prelude = f'''#include <cstdint>
#include "{tile_header}"
namespace mellum16 {{ struct DeviceMatrix {{ const unsigned char *data = nullptr; const unsigned char *scales = nullptr;
  const float *divisor = nullptr; int rows = 0, cols = 0, format = 0; const std::uint16_t *suh = nullptr; const std::uint16_t *svh = nullptr; }}; }}
'''
    else:
        prelude = "#define PADRA_B200_BIND_STANDALONE\n"
    source.write_text(prelude + f'''#include "{ROOT / "padra_b200" / "host" / "bind.hpp"}"
using namespace padra_b200_bind;
void all(const mellum16::DeviceMatrix *m, mellum16::exl3_masked_schedule::Tile *tiles, int *i, float *f, unsigned *u,
         unsigned short *h, __half *w, void *ws, cudaStream_t s) {{
  DecodeLaunch(m, 0, 0, i, f, f, f, 8, i, s, u, f, 4);
  MtpUnion(i, u, i, 5, i, i, i, s);
  MtpLaunch(m, 0, 0, u, i, 5, f, f, f, i, s, i, i, 4);
  SiluBuild(h, s);
  SiluActivate(f, f, h, 8, i, s);
  Combine(f, f, f, i, 1, s);
  Group(i, i, i, 4, i, s);
  Schedule(i, tiles, i, 4, i, s);
  PrefillLaunch(m, 0, 0, i, i, i, tiles, i, f, h, h, h, h, w, 4, i, s, u, true, 4);
  CombinePacked(f, h, f, 4, i, true, s);
  ExpertLaunch(m, 0, 0, i, f, f, f, f, 1, i, s, false, u, 4);
  DecodeLayer(m, 0, i, f, f, f, 1, 4, h, ws, 0, i, s);
  DraftExpertLayer(m, i, f, f, f, h, ws, 0, i, s);
}}
''')
    cuda_include = "/usr/local/cuda/include"
    out = subprocess.run(["g++", "-std=c++20", "-fsyntax-only", "-Wall", f"-I{cuda_include}", str(source)], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
