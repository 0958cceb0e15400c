"""CPU oracle for the EXL3 MoE expert path -- Python side.  TEST INFRASTRUCTURE ONLY.

Two things live here:

* ``COracle`` / ``RefWeight`` / ``RefKernels``: ctypes loaders for ``libexl3_oracle.so`` (the plain-C
  restatement, ``exl3_oracle.c``), ``_ref/libref_weight.so`` (the reference's own scalar decoder source
  compiled for the host) and ``_ref/libref_kernels.so`` (the reference's own CUDA kernels compiled for
  sm_100a).  ``oracle/Makefile`` builds all three.
* a vectorised numpy twin of the trellis decoder and of the Hadamard/BF16 helpers, written independently
  of the C code so that the two restatements check each other.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module; the product
package (``padra_b200``) never does.  Reference citations are paths inside the reference checkout.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
FORMAT_OF_RATE = {3: 6, 4: 3, 6: 5}  # src/cuda/device_matrix.cuh:30-44
RATE_OF_FORMAT = {v: k for k, v in FORMAT_OF_RATE.items()}


class Matrix(C.Structure):
    """src/cuda/device_matrix.cuh:6-13 -- seven fields, 56 bytes."""

    _fields_ = [
        ("data", C.c_void_p),
        ("scales", C.c_void_p),
        ("divisor", C.c_void_p),
        ("rows", C.c_int),
        ("cols", C.c_int),
        ("format", C.c_int),
        ("suh", C.c_void_p),
        ("svh", C.c_void_p),
    ]


assert C.sizeof(Matrix) == 56


# ----------------------------------------------------------------------------------------------
# numpy twin
# ----------------------------------------------------------------------------------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    """B(): FP32 -> BF16 (nearest even) -> FP32.  src/cuda/inference.cu:52-54"""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    r = np.where(nan, 0x7FFF0000, r)  # canonical NaN, as __float2bfloat16_rn
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def tile_permutation() -> np.ndarray:
    """perm[input_in_tile, output_in_tile] -> position in the tile.  src/cuda/expert_exl3.cuh:4-7"""
    i = np.arange(16)[:, None]
    o = np.arange(16)[None, :]
    return ((o & 7) * 4 + ((i & 7) >> 1)) * 8 + np.where(o >= 8, 4, 0) + np.where(i >= 8, 2, 0) + (i & 1)


def mul1_bits(state: np.ndarray) -> np.ndarray:
    """FP16 bit patterns of the 'mul1' codebook for 16-bit states.  src/cuda/expert_exl3.cuh:19-21

    hfma(1024+s, 0x1eee, 0xc931) is one rounding of an exactly representable double."""
    h = (state.astype(np.uint64) * 0x83DCD12D) & 0xFFFFFFFF
    s = (h & 255) + ((h >> 8) & 255) + ((h >> 16) & 255) + (h >> 24)
    a = np.array([0x1EEE], dtype=np.uint16).view(np.float16).astype(np.float64)[0]
    c = np.array([0xC931], dtype=np.uint16).view(np.float16).astype(np.float64)[0]
    exact = (1024.0 + s.astype(np.float64)) * a + c
    return exact.astype(np.float16).view(np.uint16)


def tile_states(data: np.ndarray, rate: int) -> np.ndarray:
    """All 256 cyclic 16-bit states of every tile: (tiles, 256).  src/cuda/expert_exl3.cuh:8-18"""
    words = np.ascontiguousarray(data).view("<u4").reshape(-1, 8 * rate)
    shifts = (31 - np.arange(32, dtype=np.uint32))[None, None, :]
    bits = ((words[:, :, None] >> shifts) & 1).astype(np.uint8).reshape(words.shape[0], 256 * rate)
    p = np.arange(256)[:, None]
    pos = (p * rate + rate - 16 + np.arange(16)[None, :]) % (256 * rate)
    window = bits[:, pos].astype(np.uint32)
    return (window << (15 - np.arange(16, dtype=np.uint32))[None, None, :]).sum(axis=2).astype(np.uint32)


def decode_matrix_bits(data: np.ndarray, rows: int, cols: int, rate: int) -> np.ndarray:
    """FP16 bits of every weight as an array [cols(input), rows(output)].

    Tiles are stored input-block-major: tile (ib, ob) at index ib*(rows/16)+ob.  expert_exl3.cuh:10-12"""
    st = tile_states(data, rate).reshape(cols // 16, rows // 16, 256)
    perm = tile_permutation()
    w = mul1_bits(st[:, :, perm])  # (ib, ob, i, o)
    return np.ascontiguousarray(w.transpose(0, 2, 1, 3)).reshape(cols, rows)


def hadamard128(x: np.ndarray) -> np.ndarray:
    """FP32 butterflies d=1..64 then *1/sqrt(128), over the last axis (length 128).  expert_exl3.cuh:48-55"""
    v = np.array(x, dtype=np.float32, copy=True)
    t = np.arange(128)
    for d in (1, 2, 4, 8, 16, 32, 64):
        other = v[..., t ^ d]
        v = np.where((t & d) != 0, other - v, v + other).astype(np.float32)
    return (v * np.float32(0.08838834764831845)).astype(np.float32)


def input_had(x: np.ndarray, suh_bits: np.ndarray) -> np.ndarray:
    """expert_exl3.cuh:32-59 over the last axis (multiple of 128)."""
    s = suh_bits.view(np.float16).astype(np.float32)
    v = (x.astype(np.float32) * s).astype(np.float32)
    v = hadamard128(v.reshape(*v.shape[:-1], -1, 128)).reshape(v.shape)
    return bf16_round(v)


def output_had(raw: np.ndarray, svh_bits: np.ndarray) -> np.ndarray:
    """expert_exl3.cuh:88-113"""
    s = svh_bits.view(np.float16).astype(np.float32)
    v = hadamard128(raw.astype(np.float32).reshape(*raw.shape[:-1], -1, 128)).reshape(raw.shape)
    return bf16_round((v * s).astype(np.float32))


def linear_f64(data, rows, cols, rate, suh, svh, x) -> np.ndarray:
    """One EXL3 linear with the dot product in FP64 (an accuracy yardstick, not a bit-level oracle)."""
    w = decode_matrix_bits(data, rows, cols, rate).view(np.float16).astype(np.float64)
    xt = input_had(x, suh).astype(np.float64)
    raw = (xt @ w).astype(np.float32)
    return output_had(raw, svh)


# ----------------------------------------------------------------------------------------------
# synthetic matrices in the reference's tensor layout
# ----------------------------------------------------------------------------------------------
def synthetic_matrix(rng: np.random.Generator, rows: int, cols: int, rate: int):
    """Uniform random trellis words (any bit pattern is a valid tail-biting stream) plus FP16 sign/scale
    sidecars (+-1) * U(0.5, 1.5).  Returns (data u8, suh u16, svh u16)."""
    data = rng.integers(0, 2**32, size=(cols // 16) * (rows // 16) * 8 * rate, dtype=np.uint32).view(np.uint8)
    def sidecar(n):
        v = rng.uniform(0.5, 1.5, size=n) * rng.choice([-1.0, 1.0], size=n)
        return v.astype(np.float16).view(np.uint16)
    return data, sidecar(cols), sidecar(rows)


class HostMatrices:
    """A table of host matrices shaped like the reference's descriptor table
    (index (layer*64+expert)*3+part, src/cuda/inference.cu:1599-1602), with the arrays kept alive."""

    def __init__(self, layers: int, hidden: int, inter: int, rate: int, seed: int = 0, experts: int = 64):
        self.layers, self.hidden, self.inter, self.rate, self.experts = layers, hidden, inter, rate, experts
        rng = np.random.Generator(np.random.Philox(key=seed))
        self.table = (Matrix * (layers * experts * 3))()
        self.arrays = []
        for layer in range(layers):
            for e in range(experts):
                for part in range(3):
                    rows, cols = (hidden, inter) if part == 2 else (inter, hidden)
                    data, suh, svh = synthetic_matrix(rng, rows, cols, rate)
                    self.arrays.append((data, suh, svh))
                    m = self.table[(layer * experts + e) * 3 + part]
                    m.data = data.ctypes.data
                    m.suh = suh.ctypes.data
                    m.svh = svh.ctypes.data
                    m.rows, m.cols, m.format = rows, cols, FORMAT_OF_RATE[rate]

    def get(self, layer: int, expert: int, part: int):
        return self.arrays[(layer * self.experts + expert) * 3 + part]


# ----------------------------------------------------------------------------------------------
# ctypes loaders
# ----------------------------------------------------------------------------------------------
def _f32p(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _i32p(a):
    return a.ctypes.data_as(C.POINTER(C.c_int))


class COracle:
    """libexl3_oracle.so"""

    def __init__(self, path: os.PathLike | None = None):
        self.lib = C.CDLL(str(path or HERE / "libexl3_oracle.so"))
        L = self.lib
        L.exl3_bf16_round.restype = C.c_float
        L.exl3_bf16_round.argtypes = [C.c_float]
        L.exl3_f32_to_f16_bits.restype = C.c_uint16
        L.exl3_f32_to_f16_bits.argtypes = [C.c_float]
        L.exl3_f16_bits_to_f32.restype = C.c_float
        L.exl3_f16_bits_to_f32.argtypes = [C.c_uint16]
        L.exl3_index.restype = C.c_uint
        L.exl3_index.argtypes = [C.c_uint, C.c_uint]
        L.exl3_mul1_bits.restype = C.c_uint16
        L.exl3_mul1_bits.argtypes = [C.c_uint]
        L.exl3_weight_bits.restype = C.c_uint16
        L.exl3_weight_bits.argtypes = [C.POINTER(Matrix), C.c_int, C.c_int]
        L.exl3_decode_matrix.restype = None
        L.exl3_decode_matrix.argtypes = [C.POINTER(Matrix), C.c_void_p]
        for name in ("exl3_input_had", "exl3_dot", "exl3_output_had", "exl3_linear", "exl3_linear_f16"):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = [C.POINTER(Matrix), C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.exl3_silu_rounded.restype = C.c_float
        L.exl3_silu_rounded.argtypes = [C.c_float]
        L.exl3_silu_table.argtypes = [C.c_void_p]
        L.exl3_activate.restype = C.c_int
        L.exl3_activate.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int]
        L.exl3_route.restype = C.c_int
        L.exl3_route.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_int), C.POINTER(C.c_float)]
        L.exl3_combine.restype = C.c_int
        L.exl3_combine.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int]
        L.exl3_group.restype = C.c_int
        L.exl3_group.argtypes = [C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int]
        L.exl3_schedule.restype = C.c_int
        L.exl3_schedule.argtypes = [C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int]
        L.exl3_moe_layer.restype = C.c_int
        L.exl3_moe_layer.argtypes = [C.POINTER(Matrix), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float),
                                     C.POINTER(C.c_float), C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.exl3_residual_norm.restype = C.c_int
        L.exl3_residual_norm.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_void_p, C.c_int,
                                         C.POINTER(C.c_float)]
        L.exl3_combine_norm.restype = C.c_int
        L.exl3_combine_norm.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float),
                                        C.c_void_p, C.c_int, C.POINTER(C.c_float)]
        L.exl3_set_threads.argtypes = [C.c_int]
        L.exl3_get_threads.restype = C.c_int

    @staticmethod
    def matrix(data, suh, svh, rows, cols, rate) -> Matrix:
        data, suh, svh = (np.ascontiguousarray(a) for a in (data, suh, svh))
        m = Matrix()
        m.data, m.suh, m.svh = data.ctypes.data, suh.ctypes.data, svh.ctypes.data
        m.rows, m.cols, m.format = rows, cols, FORMAT_OF_RATE[rate]
        m._keep = (data, suh, svh)  # the descriptor only holds addresses
        return m

    def decode_matrix(self, data, rows, cols, rate) -> np.ndarray:
        data = np.ascontiguousarray(data)
        m = Matrix()
        m.data, m.rows, m.cols, m.format = data.ctypes.data, rows, cols, FORMAT_OF_RATE[rate]
        out = np.empty((cols, rows), dtype=np.uint16)
        self.lib.exl3_decode_matrix(C.byref(m), out.ctypes.data)
        return out

    def linear(self, m: Matrix, x: np.ndarray, f16_form: bool = False):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(m.rows, dtype=np.float32)
        fn = self.lib.exl3_linear_f16 if f16_form else self.lib.exl3_linear
        bad = fn(C.byref(m), _f32p(x), _f32p(y))
        return y, bad

    def input_had(self, m: Matrix, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(m.cols, dtype=np.float32)
        bad = self.lib.exl3_input_had(C.byref(m), _f32p(x), _f32p(y))
        return y, bad

    def route(self, logits: np.ndarray):
        logits = np.ascontiguousarray(logits, dtype=np.float32).reshape(-1, 64)
        ids = np.empty((logits.shape[0], 8), dtype=np.int32)
        w = np.empty((logits.shape[0], 8), dtype=np.float32)
        bad = 0
        for t in range(logits.shape[0]):
            bad |= self.lib.exl3_route(_f32p(logits[t]), _i32p(ids[t]), _f32p(w[t]))
        return ids, w, bad

    def swiglu(self, gate: np.ndarray, up: np.ndarray) -> np.ndarray:
        """B(silu_bf16(gate) * up) element by element (src/cuda/inference.cu:575-579); returns a new array."""
        act = np.array(gate, dtype=np.float32, copy=True).reshape(-1)
        up = np.ascontiguousarray(up, dtype=np.float32).reshape(-1)
        bad = self.lib.exl3_activate(_f32p(act), _f32p(up), act.size)
        assert not bad, "non-finite SwiGLU input"
        return act.reshape(np.shape(gate))

    def combine(self, x: np.ndarray, down: np.ndarray, weights: np.ndarray):
        """x[t] = B(x[t] + sum over the eight slots) for every token (src/cuda/inference.cu:580-594).
        x [tokens][hidden], down [tokens][8][hidden], weights [tokens][8]; returns (new x, bad)."""
        out = np.array(x, dtype=np.float32, copy=True)
        tokens, hidden = out.shape
        down = np.ascontiguousarray(down, dtype=np.float32).reshape(tokens, 8, hidden)
        weights = np.ascontiguousarray(weights, dtype=np.float32).reshape(tokens, 8)
        bad = 0
        for t in range(tokens):
            bad |= self.lib.exl3_combine(_f32p(out[t]), _f32p(down[t]), _f32p(weights[t]), hidden)
        return out, bad

    def residual_norm(self, x, residual, weight_bits):
        """Rows of ResidualPostNormWideExact (src/cuda/residual_norm_wide_exact.cuh:84-131): returns (x, normalized,
        stats[rows][2], bad); residual may be None; weight_bits are BF16 bit patterns [hidden]."""
        out = np.array(x, dtype=np.float32, copy=True)
        rows, hidden = out.shape
        res = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32).reshape(rows, hidden)
        weight_bits = np.ascontiguousarray(weight_bits, dtype=np.uint16)
        normalized, stats, bad = np.empty_like(out), np.empty((rows, 2), np.float32), 0
        for r in range(rows):
            bad |= self.lib.exl3_residual_norm(_f32p(out[r]), None if res is None else _f32p(res[r]), _f32p(normalized[r]),
                                               weight_bits.ctypes.data, hidden, _f32p(stats[r]))
        return out, normalized, stats, bad

    def combine_norm(self, x, down, routing, weight_bits):
        """Rows of combine_norm_exact::CombineNorm<false> (src/cuda/combine_norm_exact.cuh:7-68): x [rows][hidden],
        down [rows][8][hidden], routing [rows][8]; returns (x, normalized, stats, bad)."""
        out = np.array(x, dtype=np.float32, copy=True)
        rows, hidden = out.shape
        down = np.ascontiguousarray(down, dtype=np.float32).reshape(rows, 8, hidden)
        routing = np.ascontiguousarray(routing, dtype=np.float32).reshape(rows, 8)
        weight_bits = np.ascontiguousarray(weight_bits, dtype=np.uint16)
        normalized, stats, bad = np.empty_like(out), np.empty((rows, 2), np.float32), 0
        for r in range(rows):
            bad |= self.lib.exl3_combine_norm(_f32p(out[r]), _f32p(down[r]), _f32p(routing[r]), _f32p(normalized[r]),
                                              weight_bits.ctypes.data, hidden, _f32p(stats[r]))
        return out, normalized, stats, bad

    def silu_table(self) -> np.ndarray:
        t = np.empty(65536, dtype=np.uint16)
        self.lib.exl3_silu_table(t.ctypes.data)
        return t

    def group(self, ids: np.ndarray, tokens: int):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        groups = np.full(64 * tokens, -1, dtype=np.int32)
        counts = np.zeros(64, dtype=np.int32)
        bad = self.lib.exl3_group(_i32p(ids), _i32p(groups), _i32p(counts), tokens)
        return groups, counts, bad

    def schedule(self, counts: np.ndarray, tokens: int):
        counts = np.ascontiguousarray(counts, dtype=np.int32)
        cap = (tokens * 8 + 31) // 32 + 64
        tiles = np.zeros((cap, 3), dtype=np.int32)
        n = C.c_int(0)
        bad = self.lib.exl3_schedule(_i32p(counts), _i32p(tiles), C.byref(n), tokens)
        return tiles[: n.value], bad

    def moe_layer(self, table, layer, ids, weights, x, hidden, inter, f16_form=False, capture=False):
        """Returns (x_out, bad[, captures]); x is [tokens, hidden] FP32 holding BF16 values."""
        ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
        weights = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
        out = np.array(x, dtype=np.float32, copy=True).reshape(-1, hidden)
        tokens = out.shape[0]
        caps = [None] * 4
        ptrs = [None] * 4
        if capture:
            caps = [np.empty((tokens * 8, inter), np.float32) for _ in range(3)] + [np.empty((tokens * 8, hidden), np.float32)]
            ptrs = [c.ctypes.data for c in caps]
        bad = self.lib.exl3_moe_layer(table, layer, _i32p(ids), _f32p(weights), _f32p(out), tokens, hidden, inter,
                                      int(f16_form), *ptrs)
        return (out, bad, caps) if capture else (out, bad)


class RefWeight:
    """_ref/libref_weight.so: the reference's Index/Weight text (src/cuda/expert_exl3.cuh:4-22) on the host."""

    def __init__(self, path: os.PathLike | None = None):
        self.lib = C.CDLL(str(path or HERE / "_ref" / "libref_weight.so"))
        self.lib.ref_index.restype = C.c_uint
        self.lib.ref_index.argtypes = [C.c_uint, C.c_uint]
        self.lib.ref_weight.restype = C.c_float
        self.lib.ref_weight.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        self.lib.ref_decode_matrix.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]

    @staticmethod
    def available() -> bool:
        return (HERE / "_ref" / "libref_weight.so").exists()

    def decode_matrix(self, data, rows, cols, rate) -> np.ndarray:
        data = np.ascontiguousarray(data)
        out = np.empty((cols, rows), dtype=np.float32)
        self.lib.ref_decode_matrix(data.ctypes.data, rows, cols, FORMAT_OF_RATE[rate], out.ctypes.data)
        return out


def ref_kernels_path() -> Path:
    return HERE / "_ref" / "libref_kernels.so"


class RefKernels:
    """_ref/libref_kernels.so: the reference's own CUDA kernels (sm_100a build).  Arguments are raw device
    addresses (ints); see oracle/ref_kernels_post.h for what each entry launches."""

    def __init__(self, path: os.PathLike | None = None):
        self.lib = C.CDLL(str(path or ref_kernels_path()))
        p, i = C.c_void_p, C.c_int
        sig = {
            "ref_decode_dual": [p, i, i, p, p, p, p, i, p, p, i, i],
            "ref_decode_dual_launch": [p, i, i, p, p, p, p, i, p, p, i],
            "ref_simt_linear": [p, i, i, p, p, p, p, p, i, p, p, i, i],
            "ref_mtp_build_union": [p, p, p, i, p, p, p, p],
            "ref_mtp_projection": [p, i, i, p, p, i, p, p, p, p, p, p, p, i, i],
            "ref_group": [p, p, p, i, p, p],
            "ref_schedule": [p, p, p, i, p, p],
            "ref_prefill_launch": [p, i, i, p, p, p, p, p, p, p, p, p, p, p, i, p, p, i],
            "ref_prefill_generic": [p, i, i, p, p, p, p, p, p, p, p, p, p, p, i, p, p, i, i, i],
            "ref_silu_build": [p, p],
            "ref_silu_activate": [p, p, p, i, p, p],
            "ref_combine": [p, p, p, i, p, p],
            "ref_combine_packed": [p, p, p, i, p, i, p],
            "ref_route": [p, p, p, i, p, p],
            "ref_route_rank_exact": [p, p, p, i, p, p],
            "ref_residual_post_norm": [p, p, p, p, p, p, i, p],
            "ref_activate": [p, p, i, p],
        }
        for name, args in sig.items():
            f = getattr(self.lib, name)
            f.argtypes = args
            f.restype = i

    @staticmethod
    def available() -> bool:
        return ref_kernels_path().exists()

    def __getattr__(self, name):
        fn = getattr(self.lib, name)

        def call(*args):
            status = fn(*args)
            if status != 0:
                raise RuntimeError(f"{name}: CUDA error {status}")

        return call
