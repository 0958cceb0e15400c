"""Reader and writer of the EXL3 expert tensors of a compiled-model artifact (manifest.json + weights.bin).

The Python twin of padra_b200/host/artifact.cpp, used by the tests and by ExpertTable.save_artifact / from_artifact.
Format: the reference's (src/model/compiled.cpp:91-216): per tensor `shape` [rows, cols], `format` "EXL3_K{3,4,6}",
`codebook` "mul1", `hadamard_block` 128 and the byte regions `packed`, `suh`, `svh` of the payload, each starting on a
256-byte boundary, back to back in offset order, accounting for every payload byte; the payload's SHA-256 is recorded.
Only the expert tensors are handled (model.layers.<L>.mlp.experts.<E>.{gate,up,down}_proj.weight).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass
from pathlib import Path

import numpy as np

PARTS = ("gate", "up", "down")
FORMAT_OF_RATE = {3: 6, 4: 3, 6: 5}  # src/cuda/device_matrix.cuh:30-44


class ArtifactError(ValueError):
    pass


def _require(ok: bool, what: str) -> None:
    if not ok:
        raise ArtifactError(what)


def profile_of_rate(rate: int) -> str:
    _require(rate in FORMAT_OF_RATE, "unsupported EXL3 rate")
    return f"mellum16-exl3-k{rate}-fp8-bf16-v1"  # src/model/compiled.h:11-14


def expert_tensor_name(layer: int, expert: int, part: int) -> str:
    return f"model.layers.{layer}.mlp.experts.{expert}.{PARTS[part]}_proj.weight"  # src/cuda/inference.cu:1599-1602


@dataclass
class Tensor:
    name: str
    rows: int
    cols: int
    rate: int
    packed: tuple[int, int]  # (offset, bytes)
    suh: tuple[int, int]
    svh: tuple[int, int]


@dataclass
class Artifact:
    directory: Path
    profile: str
    rate: int
    weights_bytes: int
    weights_sha256: str
    tensors: dict[str, Tensor]
    layers: int

    def payload(self) -> np.ndarray:
        return np.fromfile(self.directory / "weights.bin", dtype=np.uint8)


def write(directory, rate: int, tensors) -> None:
    """tensors: iterable of (name, rows, cols, packed u8[rows*cols*rate/8], suh u16[cols], svh u16[rows])."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    payload = bytearray()
    table = {}
    for name, rows, cols, packed, suh, svh in tensors:
        _require(rows >= 128 and cols >= 128 and rows % 128 == 0 and cols % 128 == 0, "wrong tensor shape")
        regions = {}
        for part, data, want in (("packed", packed, rows * cols * rate // 8), ("suh", suh, 2 * cols), ("svh", svh, 2 * rows)):
            raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
            _require(raw.size == want, f"{name}: region {part} has {raw.size} bytes, expected {want}")
            payload.extend(b"\0" * (-len(payload) % 256))
            regions[part] = {"offset": len(payload), "bytes": want}
            payload.extend(raw.tobytes())
        table[name] = {"shape": [rows, cols], "format": f"EXL3_K{rate}", "codebook": "mul1", "hadamard_block": 128, "regions": regions}
    _require(bool(table), "nothing to write")
    (directory / "weights.bin").write_bytes(bytes(payload))
    manifest = {"schema_version": 1, "profile": profile_of_rate(rate), "weights_file": "weights.bin", "weights_bytes": len(payload),
                "weights_sha256": hashlib.sha256(bytes(payload)).hexdigest(), "tensors": table}
    (directory / "manifest.json").write_text(json.dumps(manifest, indent=1))


def load(directory, verify_payload: bool = True, experts_only: bool = False) -> Artifact:
    directory = Path(directory)
    for name in ("manifest.json", "weights.bin"):
        p = directory / name
        _require(p.is_file() and not p.is_symlink(), "artifact file must be regular and not a symlink")
    _require((directory / "manifest.json").stat().st_size < 4 << 20, "manifest too large")
    v = json.loads((directory / "manifest.json").read_text())
    _require(v.get("schema_version") == 1, "unsupported manifest schema")
    profile = v.get("profile")
    rate = next((r for r in FORMAT_OF_RATE if profile == profile_of_rate(r)), 0)
    _require(rate != 0, "unsupported precision/math profile")
    _require(v.get("weights_file") == "weights.bin", "unsafe weights path")
    nbytes = v.get("weights_bytes")
    _require(isinstance(nbytes, int) and 0 < nbytes < 12 << 30, "invalid artifact byte budget")
    _require((directory / "weights.bin").stat().st_size == nbytes, "truncated or oversized weight payload")
    sha = v.get("weights_sha256")
    _require(isinstance(sha, str) and len(sha) == 64 and all(c in "0123456789abcdef" for c in sha), "invalid weight hash")
    tensors, ranges, layers = {}, [], 0
    for name, t in v["tensors"].items():
        if ".experts." not in name:
            _require(experts_only, "not an expert tensor (pass experts_only to skip others)")
            continue
        shape = t["shape"]
        _require(len(shape) == 2, "wrong tensor rank")
        rows, cols = shape
        _require(rows >= 128 and cols >= 128 and rows % 128 == 0 and cols % 128 == 0, "wrong tensor shape")
        _require(t["format"] == f"EXL3_K{rate}", "tensor precision does not match selected hybrid")
        _require(t["codebook"] == "mul1" and t["hadamard_block"] == 128, "unsupported EXL3 codec/transform")
        regions = t["regions"]
        _require(len(regions) == 3, "unknown/missing weight regions")
        got = {}
        for part, want in (("packed", rows * cols * rate // 8), ("suh", 2 * cols), ("svh", 2 * rows)):
            r = regions[part]
            off, n = r["offset"], r["bytes"]
            _require(off % 256 == 0 and n == want and off <= nbytes and n <= nbytes - off, "invalid region range/alignment/bytes")
            got[part] = (off, n)
            ranges.append((off, n))
        tensors[name] = Tensor(name, rows, cols, rate, got["packed"], got["suh"], got["svh"])
        layers = max(layers, int(name.split(".")[2]) + 1)
    _require(bool(tensors), "incomplete/extra tensor inventory")
    if not experts_only:
        cursor = 0
        for off, n in sorted(ranges):
            _require(off == (cursor + 255) // 256 * 256, "overlapping/noncanonical weight regions")
            cursor = off + n
        _require(cursor == nbytes, "unaccounted payload bytes")
    art = Artifact(directory, profile, rate, nbytes, sha, tensors, layers)
    if verify_payload:
        payload = art.payload()
        _require(hashlib.sha256(payload.tobytes()).hexdigest() == sha, "weight SHA-256 mismatch")
        for t in tensors.values():
            for off, n in (t.suh, t.svh):
                side = payload[off:off + n].view(np.uint16)
                _require(not ((side & 0x7C00) == 0x7C00).any(), "nonfinite EXL3 FP16 sidecar")
                _require(not ((side & 0x7FFF) == 0).any(), "zero EXL3 sidecar")
    return art
