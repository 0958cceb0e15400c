"""CPU tests of the drop-in boundary: the library builds for sm_100a, loads, and exports exactly the
symbols include/padra_b200.h declares.  No kernel is launched here."""
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    from padra_b200 import binding, build

    build.build()
    return binding.load()


def declared_symbols():
    text = (ROOT / "include" / "padra_b200.h").read_text()
    return re.findall(r"PADRA_API\s+[\w\s\*]+?\b(padra_\w+)\s*\(", text)


def test_header_and_binding_agree(lib):
    from padra_b200 import binding

    names = declared_symbols()
    assert len(names) >= 15 and len(set(names)) == len(names)
    assert set(names) == set(binding.SIGNATURES), set(names) ^ set(binding.SIGNATURES)
    for n in names:
        assert hasattr(lib, n)


def test_exports_only_the_abi(lib):
    from padra_b200 import binding

    out = subprocess.check_output(["nm", "-D", "--defined-only", str(binding.LIB_PATH)], text=True)
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    assert exported == set(declared_symbols()), exported ^ set(declared_symbols())


def test_descriptor_layout_matches_reference_struct():
    import ctypes as C

    from oracle.exl3_oracle import Matrix
    from padra_b200.experts import DESCRIPTOR

    assert DESCRIPTOR.itemsize == C.sizeof(Matrix) == 56
    for name in ("data", "scales", "divisor", "rows", "cols", "format", "suh", "svh"):
        assert DESCRIPTOR.fields[name][1] == getattr(Matrix, name).offset


def test_host_side_argument_checks(lib):
    from padra_b200 import binding as B

    assert lib.padra_version() >= 100
    assert lib.padra_status_string(B.INVALID_ARGUMENT) == b"invalid argument"
    assert lib.padra_exl3_moe_decode_workspace_bytes(0, 2048, 1024) == 0
    assert lib.padra_exl3_moe_decode_workspace_bytes(17, 2048, 1024) == 0
    n = lib.padra_exl3_moe_decode_workspace_bytes(1, 2048, 1024)
    assert n >= 8 * (1024 * 2 + 2048) * 4
    # null pointers / bad sizes are refused on the host before any launch
    assert lib.padra_exl3_decode_launch(None, 0, 0, None, None, None, None, 8, None, None, None, None, 4, 2048, 1024) == B.INVALID_ARGUMENT
    assert lib.padra_exl3_decode_launch(None, 0, 0, None, None, None, None, 8, None, None, None, None, 5, 2048, 1024) == B.UNSUPPORTED
    assert lib.padra_exl3_prefill_launch(None, 0, 0, *([None] * 11), 3, None, None, None, 0, 4, 2048, 1024) == B.INVALID_ARGUMENT  # T < 4
    assert lib.padra_expert_group(None, None, None, 4, None, None) == B.INVALID_ARGUMENT
    assert lib.padra_exl3_moe_decode_layer(None, 0, None, None, None, None, 1, 4, 2048, 1024, None, None, 0, None, None) == B.INVALID_ARGUMENT


def test_missing_library_fails_loudly(tmp_path):
    from padra_b200 import binding

    with pytest.raises(FileNotFoundError):
        binding.load(tmp_path / "libpadra_b200.so")


def test_graft_entry_build_runs():
    code = "import __graft_entry__ as g; g.build(); print('built')"
    out = subprocess.check_output([sys.executable, "-c", code], cwd=ROOT, text=True)
    assert "built" in out
