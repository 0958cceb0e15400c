"""ctypes binding of the C ABI declared in include/padra_b200.h.

The library is the product; this module only hands it device pointers (torch is used for device memory and
streams, nothing else).  There is no CPU path: if the shared library is missing, loading fails loudly.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libpadra_b200.so"

OK, INVALID_ARGUMENT, UNSUPPORTED, RESOURCE_EXHAUSTED, INTERNAL = 0, 1, 5, 6, 8
FORMAT_OF_RATE = {3: 6, 4: 3, 6: 5}  # reference: src/cuda/device_matrix.cuh:30-44
MAX_DECODE_ROWS = 16

_p = C.c_void_p
_i = C.c_int

# name -> argument types, in the order of include/padra_b200.h
SIGNATURES = {
    "padra_version": ([], _i),
    "padra_status_string": ([_i], C.c_char_p),
    "padra_device_supported": ([], _i),
    "padra_exl3_decode_launch": ([_p, _i, _i, _p, _p, _p, _p, _i, _p, _p, _p, _p, _i, _i, _i], _i),
    "padra_mtp_build_union": ([_p, _p, _p, _i, _p, _p, _p, _p, _i], _i),
    "padra_mtp_experts_launch": ([_p, _i, _i, _p, _p, _i, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i], _i),
    "padra_exl3_silu_build": ([_p, _p], _i),
    "padra_exl3_silu_activate": ([_p, _p, _p, _i, _p, _p], _i),
    "padra_combine": ([_p, _p, _p, _p, _i, _i, _p], _i),
    "padra_combine_packed": ([_p, _p, _p, _i, _p, _i, _i, _p], _i),
    "padra_expert_group": ([_p, _p, _p, _i, _p, _p], _i),
    "padra_exl3_schedule": ([_p, _p, _p, _i, _p, _p], _i),
    "padra_exl3_prefill_launch": ([_p, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _i, _i, _i, _i], _i),
    "padra_exl3_expert_launch": ([_p, _i, _i, _p, _p, _p, _p, _p, _i, _p, _p, _i, _i, _i], _i),
    "padra_exl3_moe_decode_workspace_bytes": ([_i, _i, _i], C.c_size_t),
    "padra_exl3_moe_decode_workspace_init": ([_p, C.c_size_t, _p], _i),
    "padra_ep_exchange_bytes": ([_i, _i, _i, _p], C.c_size_t),
    "padra_ep_dispatch": ([_p, _p, _p, _p, _p, _i, _i, _i, _i, _i, C.c_uint, _p, _p], _i),
    "padra_ep_wait": ([_p, _i, _i, _i, _i, C.c_uint, _p, _p], _i),
    "padra_ep_set_wait_limit_ms": ([_i], _i),
    "padra_prefill_set_reserved_sms": ([_i], _i),
    "padra_ep_group_received": ([_p, _i, _i, _i, _p, _p, _i, _p, _p], _i),
    "padra_ep_return": ([_p, _p, _i, _i, _i, _i, C.c_uint, _p, _p, _i, _i, _i], _i),
    "padra_ep_down_return": ([_p, _i, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, C.c_uint, _p, _p, _i, _i, _i], _i),
    "padra_ep_plan": ([_p, _p, _p, _p, _p, _p, _i, _i, _p, _p], _i),
    "padra_ep_pack_rows": ([_p, _p, _p, _i, _i, _p, _p], _i),
    "padra_ep_group_rows": ([_p, _p, _p, _i, _i, _p, _p], _i),
    "padra_exl3_prefill_rows_launch": ([_p, _i, _i, _p, _p, _i, _i, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i], _i),
    "padra_exl3_prefill_gate_up_launch": ([_p, _i, _p, _p, _p, _p, _p, _p, _i, _p, _p, _i, _i, _i], _i),
    "padra_exl3_prefill_rows_gate_up_launch": ([_p, _i, _p, _p, _i, _i, _p, _p, _p, _p, _p, _p, _i, _i, _i], _i),
    "padra_ep_combine": ([_p, _p, _p, _p, _i, _p, _i, _i, _p], _i),
    "padra_exl3_moe_decode_layer_static": ([_p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, _p], _i),
    "padra_exl3_moe_decode_layer_launches": ([_p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, C.c_size_t, _p, _p, C.c_uint], _i),
    "padra_exl3_moe_decode_layer": ([_p, _i, _p, _p, _p, _p, _i, _i, _i, _i, _p, _p, C.c_size_t, _p, _p], _i),
    "padra_exl3_decode_weights": ([_p, _p, _i, _i, _i, _p, _p], _i),
    "padra_exl3_decode_weights_tensor": ([_p, _p, _i, _i, _i, _p, _p], _i),
    "padra_route": ([_p, _p, _p, _i, _p, _p], _i),
    "padra_route_group_schedule": ([_p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p], _i),
    "padra_residual_norm": ([_p, _p, _p, _p, _i, _i, _p, _p, _p], _i),
    "padra_combine_norm": ([_p, _p, _p, _p, _p, _i, _i, _p, _p, _p], _i),
    "padra_codec_ceiling_launch": ([_i, _i, _i, _i, _p, _p], _i),
}


class PadraError(RuntimeError):
    def __init__(self, status: int, what: str):
        super().__init__(f"{what}: status {status}")
        self.status = status


_lib = None


def load(path: Path | None = None) -> C.CDLL:
    """Loads libpadra_b200.so and types every entry point.  Raises if the library is absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    target = Path(path or LIB_PATH)
    if not target.exists():
        raise FileNotFoundError(
            f"{target} is missing: build it with `python -m padra_b200.build` (nvcc, sm_100a); there is no fallback path")
    lib = C.CDLL(str(target))
    for name, (argtypes, restype) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export a declared symbol
        fn.argtypes = argtypes
        fn.restype = restype
    if path is None:
        _lib = lib
    return lib


def ptr(t) -> int | None:
    """Device (or host) address of a torch tensor, None for None."""
    return None if t is None else t.data_ptr()


def stream_handle(stream=None) -> int:
    import torch

    return (stream or torch.cuda.current_stream()).cuda_stream


def check(status: int, what: str) -> None:
    if status != OK:
        raise PadraError(status, what)
