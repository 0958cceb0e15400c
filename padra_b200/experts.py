"""Expert weight tables in device memory and Python-side wrappers of the library's entry points.

`ExpertTable` lays the packed EXL3 tensors of `layers x 64 experts x {gate, up, down}` out in one device arena
(each region 256-byte aligned, like the reference artifact: src/model/compiled.cpp:187-216) and builds the
descriptor table the kernels index as (layer*64+expert)*3+part (reference: src/cuda/inference.cu:1599-1602).
`Workspace` owns the caller-side buffers the entry points expect; the wrappers only pass pointers through.
"""
from __future__ import annotations

import numpy as np
import torch

from . import binding as B

DESCRIPTOR = np.dtype(
    {
        "names": ["data", "scales", "divisor", "rows", "cols", "format", "suh", "svh"],
        "formats": ["<u8", "<u8", "<u8", "<i4", "<i4", "<i4", "<u8", "<u8"],
        "offsets": [0, 8, 16, 24, 28, 32, 40, 48],
        "itemsize": 56,
    }
)
EXPERTS, TOPK = 64, 8


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class ExpertTable:
    """Packed expert weights of `layers` MoE layers in one device arena plus the descriptor table."""

    def __init__(self, layers: int, hidden: int, inter: int, rate: int, device="cuda"):
        assert rate in B.FORMAT_OF_RATE and hidden % 128 == 0 and inter % 128 == 0
        self.layers, self.hidden, self.inter, self.rate = layers, hidden, inter, rate
        self.device = torch.device(device)
        self.packed_bytes = hidden * inter * rate // 8
        # per matrix: packed | suh (2*cols) | svh (2*rows)
        self.region = {}
        at = 0
        for part in range(3):
            rows, cols = self.shape(part)
            p = at
            at += _align(self.packed_bytes)
            s = at
            at += _align(2 * cols)
            v = at
            at += _align(2 * rows)
            self.region[part] = (p, s, v)
        self.expert_bytes = at
        self.total_bytes = layers * EXPERTS * self.expert_bytes
        self.arena = torch.empty(self.total_bytes, dtype=torch.uint8, device=self.device)
        self.descriptors = None  # device uint8 [layers*64*3*56]
        self._bound = None  # (layer, expert, part) -> (packed, suh, svh) offsets when the arena is an artifact's payload

    def shape(self, part: int) -> tuple[int, int]:
        """(rows = outputs, cols = inputs) of part 0 gate, 1 up, 2 down."""
        return (self.hidden, self.inter) if part == 2 else (self.inter, self.hidden)

    def offsets(self, layer: int, expert: int, part: int) -> tuple[int, int, int]:
        if self._bound is not None:
            return self._bound[layer, expert, part]
        base = (layer * EXPERTS + expert) * self.expert_bytes
        p, s, v = self.region[part]
        return base + p, base + s, base + v

    def algorithmic_bytes_per_expert(self) -> int:
        """Packed words of the three matrices plus their FP16 sidecars."""
        return 3 * self.packed_bytes + 2 * 2 * (self.hidden + self.inter) + 2 * (self.inter + self.hidden)

    # ---- artifacts (manifest.json + weights.bin; src/model/compiled.cpp:91-216) --------------------------------
    def save_artifact(self, directory) -> None:
        """Writes the table's tensors as an artifact directory.  The arena already has the artifact's canonical layout
        (per matrix packed | suh | svh, each region on a 256-byte boundary), so the payload is the arena's bytes."""
        from . import artifact

        def tensors():
            for layer in range(self.layers):
                for e in range(EXPERTS):
                    for part in range(3):
                        rows, cols = self.shape(part)
                        yield (artifact.expert_tensor_name(layer, e, part), rows, cols, *self.host_matrix(layer, e, part))

        artifact.write(directory, self.rate, tensors())

    @classmethod
    def from_artifact(cls, directory, device="cuda", verify_payload: bool = True) -> "ExpertTable":
        """Uploads an artifact's payload as the arena and binds the descriptor table to its regions, wherever the
        manifest puts them (the binder of src/cuda/device_matrix.cuh:14-66)."""
        from . import artifact

        art = artifact.load(directory, verify_payload=verify_payload)
        gate = art.tensors[artifact.expert_tensor_name(0, 0, 0)]
        table = cls.__new__(cls)
        table.layers, table.hidden, table.inter, table.rate = art.layers, gate.cols, gate.rows, art.rate
        table.device = torch.device(device)
        table.packed_bytes = table.hidden * table.inter * table.rate // 8
        table.region, table.expert_bytes, table.total_bytes = None, None, art.weights_bytes
        table.arena = torch.from_numpy(art.payload()).to(table.device)
        table._bound = {}
        d = np.zeros(art.layers * EXPERTS * 3, dtype=DESCRIPTOR)
        base = table.arena.data_ptr()
        for layer in range(art.layers):
            for e in range(EXPERTS):
                for part in range(3):
                    t = art.tensors[artifact.expert_tensor_name(layer, e, part)]
                    assert (t.rows, t.cols) == table.shape(part), "artifact mixes expert shapes"
                    table._bound[layer, e, part] = (t.packed[0], t.suh[0], t.svh[0])
                    row = d[(layer * EXPERTS + e) * 3 + part]
                    row["data"], row["suh"], row["svh"] = base + t.packed[0], base + t.suh[0], base + t.svh[0]
                    row["rows"], row["cols"], row["format"] = t.rows, t.cols, B.FORMAT_OF_RATE[art.rate]
        table.host_descriptors = d
        table.descriptors = torch.from_numpy(d.view(np.uint8).copy()).to(table.device)
        return table

    def finalize(self) -> "ExpertTable":
        """(Re)builds the device descriptor table from the arena address."""
        n = self.layers * EXPERTS * 3
        d = np.zeros(n, dtype=DESCRIPTOR)
        base = self.arena.data_ptr()
        idx = np.arange(n)
        part = idx % 3
        matrix_base = base + (idx // 3).astype(np.uint64) * np.uint64(self.expert_bytes)
        for q in range(3):
            sel = part == q
            p, s, v = self.region[q]
            rows, cols = self.shape(q)
            d["data"][sel] = matrix_base[sel] + np.uint64(p)
            d["suh"][sel] = matrix_base[sel] + np.uint64(s)
            d["svh"][sel] = matrix_base[sel] + np.uint64(v)
            d["rows"][sel], d["cols"][sel] = rows, cols
        d["format"] = B.FORMAT_OF_RATE[self.rate]
        self.host_descriptors = d
        self.descriptors = torch.from_numpy(d.view(np.uint8).copy()).to(self.device)
        return self

    def descriptor_ptr(self, layer: int = 0, expert: int = 0, part: int = 0) -> int:
        return self.descriptors.data_ptr() + ((layer * EXPERTS + expert) * 3 + part) * 56

    # ---- filling -------------------------------------------------------------------------------------
    def fill_random(self, seed: int = 0) -> "ExpertTable":
        """Seeded synthetic weights generated on the device: uniformly random trellis words (every bit pattern is
        a valid tail-biting stream) and FP16 sidecars (+-1) * U(0.5, 1.5)."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        words = self.arena.view(torch.int32)
        chunk = 1 << 26
        for at in range(0, words.numel(), chunk):
            n = min(chunk, words.numel() - at)
            words[at:at + n] = torch.randint(-(2**31), 2**31 - 1, (n,), dtype=torch.int32, device=self.device, generator=g)
        per = self.arena.view(self.layers * EXPERTS, self.expert_bytes)
        for part in range(3):
            rows, cols = self.shape(part)
            p, s, v = self.region[part]
            for off, n in ((s, cols), (v, rows)):
                mag = torch.rand((per.shape[0], n), device=self.device, generator=g) + 0.5
                sign = torch.randint(0, 2, (per.shape[0], n), device=self.device, generator=g) * 2 - 1
                side = (mag * sign).to(torch.float16)
                per[:, off:off + 2 * n] = side.view(torch.uint8)
        return self.finalize()

    def fill_from_host(self, host) -> "ExpertTable":
        """Uploads the arrays of an oracle-side host table (same shapes), so CPU and GPU see identical bytes."""
        staging = np.zeros(self.total_bytes, dtype=np.uint8)
        for layer in range(self.layers):
            for e in range(EXPERTS):
                for part in range(3):
                    data, suh, svh = host.get(layer, e, part)
                    p, s, v = self.offsets(layer, e, part)
                    staging[p:p + data.size] = data
                    staging[s:s + 2 * suh.size] = suh.view(np.uint8)
                    staging[v:v + 2 * svh.size] = svh.view(np.uint8)
        self.arena.copy_(torch.from_numpy(staging))
        return self.finalize()

    def host_matrix(self, layer: int, expert: int, part: int):
        """(data u8, suh u16, svh u16) copied back to the host, for checks against the CPU oracle."""
        rows, cols = self.shape(part)
        p, s, v = self.offsets(layer, expert, part)
        a = self.arena
        return (a[p:p + self.packed_bytes].cpu().numpy().copy(),
                a[s:s + 2 * cols].cpu().numpy().view(np.uint16).copy(),
                a[v:v + 2 * rows].cpu().numpy().view(np.uint16).copy())


class ExpertKernels:
    """Thin callers of the C ABI for one table.  Names follow the reference launchers they stand in for."""

    def __init__(self, table: ExpertTable):
        self.lib = B.load()
        self.t = table
        dev = table.device
        self.bad = torch.zeros(1, dtype=torch.int32, device=dev)
        self.table = torch.empty(65536, dtype=torch.uint16, device=dev)
        B.check(self.lib.padra_exl3_silu_build(B.ptr(self.table), B.stream_handle()), "padra_exl3_silu_build")
        self._workspace = {}

    @property
    def dims(self):
        return self.t.hidden, self.t.inter

    def reset_bad(self):
        self.bad.zero_()

    def bad_flag(self) -> int:
        return int(self.bad.item())

    # exl3_mma_dual::Launch
    def decode_launch(self, layer, part, ids, x, output, other=None, stream=None):
        pairs = ids.numel()
        st = self.lib.padra_exl3_decode_launch(self.t.descriptors.data_ptr(), layer, part, B.ptr(ids), B.ptr(x), B.ptr(output),
                                               None, pairs, B.ptr(self.bad), B.stream_handle(stream), None, B.ptr(other),
                                               self.t.rate, *self.dims)
        B.check(st, "padra_exl3_decode_launch")

    # exl3_expert::Launch
    def expert_launch(self, layer, part, ids, x, output, tokens, stream=None):
        st = self.lib.padra_exl3_expert_launch(self.t.descriptors.data_ptr(), layer, part, B.ptr(ids), B.ptr(x), B.ptr(output),
                                               None, None, tokens, B.ptr(self.bad), B.stream_handle(stream), self.t.rate,
                                               *self.dims)
        B.check(st, "padra_exl3_expert_launch")

    # mtp_experts::BuildUnion + Launch
    def build_union(self, ids, rows, slot_stride=B.MAX_DECODE_ROWS, stream=None):
        dev = self.t.device
        masks = torch.zeros(EXPERTS, dtype=torch.int32, device=dev)
        slots = torch.full((EXPERTS, slot_stride), -1, dtype=torch.int32, device=dev)
        active = torch.zeros(EXPERTS, dtype=torch.int32, device=dev)
        count = torch.zeros(1, dtype=torch.int32, device=dev)
        st = self.lib.padra_mtp_build_union(B.ptr(ids), B.ptr(masks), B.ptr(slots), rows, B.ptr(self.bad), B.ptr(active),
                                            B.ptr(count), B.stream_handle(stream), slot_stride)
        B.check(st, "padra_mtp_build_union")
        return masks, slots, active, count

    def mtp_launch(self, layer, part, union, rows, x, output, up=None, slot_stride=B.MAX_DECODE_ROWS, stream=None):
        masks, slots, active, count = union
        st = self.lib.padra_mtp_experts_launch(self.t.descriptors.data_ptr(), layer, part, B.ptr(masks), B.ptr(slots), rows,
                                               B.ptr(x), B.ptr(output), B.ptr(up), B.ptr(self.bad), B.stream_handle(stream),
                                               B.ptr(active), B.ptr(count), self.t.rate, *self.dims, slot_stride)
        B.check(st, "padra_mtp_experts_launch")

    def silu_activate(self, gate, up, stream=None):
        st = self.lib.padra_exl3_silu_activate(B.ptr(gate), B.ptr(up), B.ptr(self.table), gate.numel(), B.ptr(self.bad),
                                               B.stream_handle(stream))
        B.check(st, "padra_exl3_silu_activate")

    def combine(self, x, down, weights, rows, stream=None):
        st = self.lib.padra_combine(B.ptr(x), B.ptr(down), B.ptr(weights), B.ptr(self.bad), rows, self.t.hidden,
                                    B.stream_handle(stream))
        B.check(st, "padra_combine")

    def combine_packed(self, x, down_bits, weights, tokens, residual=True, stream=None):
        st = self.lib.padra_combine_packed(B.ptr(x), B.ptr(down_bits), B.ptr(weights), tokens, B.ptr(self.bad),
                                           int(residual), self.t.hidden, B.stream_handle(stream))
        B.check(st, "padra_combine_packed")

    # fast_expert::Group + exl3_masked::Schedule
    def group_and_schedule(self, ids, tokens, stream=None):
        dev = self.t.device
        groups = torch.full((EXPERTS * tokens,), -1, dtype=torch.int32, device=dev)
        counts = torch.zeros(EXPERTS, dtype=torch.int32, device=dev)
        capacity = (tokens * TOPK + 31) // 32 + EXPERTS
        tiles = torch.zeros((capacity, 3), dtype=torch.int32, device=dev)
        tile_count = torch.zeros(1, dtype=torch.int32, device=dev)
        B.check(self.lib.padra_expert_group(B.ptr(ids), B.ptr(groups), B.ptr(counts), tokens, B.ptr(self.bad),
                                            B.stream_handle(stream)), "padra_expert_group")
        B.check(self.lib.padra_exl3_schedule(B.ptr(counts), B.ptr(tiles), B.ptr(tile_count), tokens, B.ptr(self.bad),
                                             B.stream_handle(stream)), "padra_exl3_schedule")
        return groups, counts, tiles, tile_count

    # RouteRankExact, and the same fused with Group + Schedule
    def route(self, logits, stream=None):
        tokens = logits.shape[0]
        ids = torch.empty((tokens, TOPK), dtype=torch.int32, device=self.t.device)
        weights = torch.empty((tokens, TOPK), dtype=torch.float32, device=self.t.device)
        B.check(self.lib.padra_route(B.ptr(logits), B.ptr(ids), B.ptr(weights), tokens, B.ptr(self.bad), B.stream_handle(stream)),
                "padra_route")
        return ids, weights

    def route_group_schedule(self, logits, stream=None):
        dev, tokens = self.t.device, logits.shape[0]
        ids = torch.empty((tokens, TOPK), dtype=torch.int32, device=dev)
        weights = torch.empty((tokens, TOPK), dtype=torch.float32, device=dev)
        groups = torch.full((EXPERTS * tokens,), -1, dtype=torch.int32, device=dev)
        counts = torch.zeros(EXPERTS, dtype=torch.int32, device=dev)
        tiles = torch.zeros(((tokens * TOPK + 31) // 32 + EXPERTS, 3), dtype=torch.int32, device=dev)
        tile_count = torch.zeros(1, dtype=torch.int32, device=dev)
        if getattr(self, "_ticket", None) is None:
            self._ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        B.check(self.lib.padra_route_group_schedule(B.ptr(logits), B.ptr(ids), B.ptr(weights), B.ptr(groups), B.ptr(counts), B.ptr(tiles),
                                                    B.ptr(tile_count), tokens, B.ptr(self._ticket), B.ptr(self.bad),
                                                    B.stream_handle(stream)), "padra_route_group_schedule")
        return ids, weights, (groups, counts, tiles, tile_count)

    # ResidualPostNormWideExact / combine_norm_exact::CombineNorm
    def residual_norm(self, x, residual, normalized, weight_bits, statistics=None, stream=None):
        rows, hidden = x.shape
        B.check(self.lib.padra_residual_norm(B.ptr(x), B.ptr(residual), B.ptr(normalized), B.ptr(weight_bits), rows, hidden,
                                             B.ptr(self.bad), B.ptr(statistics), B.stream_handle(stream)), "padra_residual_norm")

    def combine_norm(self, x, down, routing, normalized, weight_bits, statistics=None, stream=None):
        rows, hidden = x.shape
        B.check(self.lib.padra_combine_norm(B.ptr(x), B.ptr(down), B.ptr(routing), B.ptr(normalized), B.ptr(weight_bits), rows, hidden,
                                            B.ptr(self.bad), B.ptr(statistics), B.stream_handle(stream)), "padra_combine_norm")

    # exl3_transport_async64::Launch / exl3_packed_activations::Launch
    def prefill_launch(self, layer, part, ids, sched, x, output_bits, gate_bits, up_bits, transformed, tokens, stream=None,
                       tensor_memory=True):
        groups, counts, tiles, tile_count = sched
        st = self.lib.padra_exl3_prefill_launch(self.t.descriptors.data_ptr(), layer, part, B.ptr(ids), B.ptr(groups),
                                                B.ptr(counts), B.ptr(tiles), B.ptr(tile_count), B.ptr(x), B.ptr(output_bits),
                                                B.ptr(gate_bits), B.ptr(up_bits), B.ptr(self.table), B.ptr(transformed),
                                                tokens, B.ptr(self.bad), B.stream_handle(stream), None, int(tensor_memory),
                                                self.t.rate, *self.dims)
        B.check(st, "padra_exl3_prefill_launch")

    def prefill_gate_up(self, layer, sched, x, gate_bits, up_bits, transformed_both, tokens, stream=None):
        """Gate and up of a chunk as one launch of the tensor-memory grouped GEMM (one list of work items)."""
        groups, counts, _, _ = sched
        st = self.lib.padra_exl3_prefill_gate_up_launch(self.t.descriptors.data_ptr(), layer, B.ptr(groups), B.ptr(counts), B.ptr(x),
                                                        B.ptr(gate_bits), B.ptr(up_bits), B.ptr(transformed_both), tokens,
                                                        B.ptr(self.bad), B.stream_handle(stream), self.t.rate, *self.dims)
        B.check(st, "padra_exl3_prefill_gate_up_launch")

    def prefill_chunk(self, layer, logits, normalized, x, tokens, stream=None):
        """A prefill chunk from the router's logits to the updated residual stream in six launches: routing + grouping +
        schedule, the gate and up input transforms, the gate+up grouped GEMM, the down input transform (SwiGLU inside), the
        down grouped GEMM, the combine.  Buffers are reused from call to call (nothing is filled in between: the
        scheduling kernel writes every count and every list entry that is read).  Returns ids and routing weights."""
        dev, (hidden, inter) = self.t.device, self.dims
        pairs = tokens * TOPK
        key = ("chunk", tokens)
        if key not in self._workspace:
            self._workspace[key] = dict(
                ids=torch.empty((tokens, TOPK), dtype=torch.int32, device=dev), weights=torch.empty((tokens, TOPK), dtype=torch.float32, device=dev),
                groups=torch.full((EXPERTS * tokens,), -1, dtype=torch.int32, device=dev), counts=torch.zeros(EXPERTS, dtype=torch.int32, device=dev),
                tiles=torch.zeros(((pairs + 31) // 32 + EXPERTS, 3), dtype=torch.int32, device=dev),
                tile_count=torch.zeros(1, dtype=torch.int32, device=dev), ticket=torch.zeros(1, dtype=torch.int32, device=dev),
                gate=torch.empty((pairs, inter), dtype=torch.uint16, device=dev), up=torch.empty((pairs, inter), dtype=torch.uint16, device=dev),
                down=torch.empty((pairs, hidden), dtype=torch.uint16, device=dev),
                transformed=torch.empty((2 * pairs, max(hidden, inter)), dtype=torch.float16, device=dev))
        w = self._workspace[key]
        st = B.stream_handle(stream)
        B.check(self.lib.padra_route_group_schedule(B.ptr(logits), B.ptr(w["ids"]), B.ptr(w["weights"]), B.ptr(w["groups"]), B.ptr(w["counts"]),
                                                    B.ptr(w["tiles"]), B.ptr(w["tile_count"]), tokens, B.ptr(w["ticket"]), B.ptr(self.bad), st),
                "padra_route_group_schedule")
        sched = (w["groups"], w["counts"], w["tiles"], w["tile_count"])
        self.prefill_gate_up(layer, sched, normalized, w["gate"], w["up"], w["transformed"], tokens, stream)
        self.prefill_launch(layer, 2, w["ids"], sched, normalized, w["down"], w["gate"], w["up"], w["transformed"], tokens, stream, True)
        self.combine_packed(x, w["down"], w["weights"], tokens, True, stream)
        return w["ids"], w["weights"]

    def prefill_layer(self, layer, ids, routing, normalized, x, tokens, stream=None, tensor_memory=True, overlap=True, merged=True):
        """gate, up, down (SwiGLU inside) and combine with residual for a prefill chunk; x updated in place.
        merged: gate and up are one launch (their work items form one list, which loads the SMs evenly).
        Otherwise, overlap: the up projection runs on a second stream beside the gate projection (its input transform
        under the gate GEMM, its first CTAs in the gate GEMM's tail); both join before the down projection."""
        dev, (hidden, inter) = self.t.device, self.dims
        pairs = tokens * TOPK
        key = ("prefill", tokens)
        if key not in self._workspace:
            self._workspace[key] = (torch.empty((pairs, inter), dtype=torch.uint16, device=dev),
                                    torch.empty((pairs, inter), dtype=torch.uint16, device=dev),
                                    torch.empty((pairs, hidden), dtype=torch.uint16, device=dev),
                                    torch.empty((pairs, max(hidden, inter)), dtype=torch.float16, device=dev),
                                    torch.empty((2 * pairs, hidden), dtype=torch.float16, device=dev))
        gate, up, down, transformed, transformed_up = self._workspace[key]
        sched = self.group_and_schedule(ids, tokens, stream)
        if merged and tensor_memory and tokens >= 4:
            self.prefill_gate_up(layer, sched, normalized, gate, up, transformed_up, tokens, stream)
            self.prefill_launch(layer, 2, ids, sched, normalized, down, gate, up, transformed, tokens, stream, tensor_memory)
        elif overlap and tensor_memory:
            main = stream or torch.cuda.current_stream()
            side = self.side_stream()
            fork, join = torch.cuda.Event(), torch.cuda.Event()
            fork.record(main)
            side.wait_event(fork)
            self.prefill_launch(layer, 1, ids, sched, normalized, up, gate, up, transformed_up, tokens, side, tensor_memory)
            join.record(side)
            self.prefill_launch(layer, 0, ids, sched, normalized, gate, gate, up, transformed, tokens, main, tensor_memory)
            main.wait_event(join)
            self.prefill_launch(layer, 2, ids, sched, normalized, down, gate, up, transformed, tokens, main, tensor_memory)
        else:
            for part, target in ((0, gate), (1, up), (2, down)):
                self.prefill_launch(layer, part, ids, sched, normalized, target, gate, up, transformed, tokens, stream, tensor_memory)
        self.combine_packed(x, down, routing, tokens, True, stream)
        return gate, up, down

    def side_stream(self):
        if getattr(self, "_side_stream", None) is None:
            self._side_stream = torch.cuda.Stream(device=self.t.device)
        return self._side_stream

    # whole decode layer
    def decode_workspace(self, tokens):
        key = ("decode", tokens)
        if key not in self._workspace:
            n = self.lib.padra_exl3_moe_decode_workspace_bytes(tokens, *self.dims)
            ws = torch.empty(n, dtype=torch.uint8, device=self.t.device)
            B.check(self.lib.padra_exl3_moe_decode_workspace_init(B.ptr(ws), n, B.stream_handle()),
                    "padra_exl3_moe_decode_workspace_init")
            self._workspace[key] = ws
        return self._workspace[key]

    def moe_decode_layer_unfused(self, layer, ids, routing, normalized, x, tokens, stream=None):
        """The same layer as separate launches through the per-part entry points (the reference's own call
        sequence: src/cuda/inference.cu:2963-2975 for one row, :3375-3392 for several)."""
        dev, (hidden, inter) = self.t.device, self.dims
        key = ("unfused", tokens)
        if key not in self._workspace:
            self._workspace[key] = (torch.empty((tokens * TOPK, inter), device=dev), torch.empty((tokens * TOPK, inter), device=dev),
                                    torch.empty((tokens * TOPK, hidden), device=dev))
        gate, up, down = self._workspace[key]
        if tokens == 1:
            self.decode_launch(layer, 0, ids, normalized, gate, up, stream)
            self.silu_activate(gate, up, stream)
            self.decode_launch(layer, 2, ids, gate, down, None, stream)
        else:
            union = self.build_union(ids, tokens, stream=stream)
            self.mtp_launch(layer, 0, union, tokens, normalized, gate, up, stream=stream)
            self.silu_activate(gate, up, stream)
            self.mtp_launch(layer, 2, union, tokens, gate, down, stream=stream)
        self.combine(x, down, routing, tokens, stream)

    def moe_decode_layer_launches(self, layer, ids, routing, normalized, x, tokens, launches, stream=None):
        ws = self.decode_workspace(tokens)
        st = self.lib.padra_exl3_moe_decode_layer_launches(self.t.descriptors.data_ptr(), layer, B.ptr(ids), B.ptr(routing),
                                                           B.ptr(normalized), B.ptr(x), tokens, self.t.rate, *self.dims,
                                                           B.ptr(self.table), B.ptr(ws), ws.numel(), B.ptr(self.bad),
                                                           B.stream_handle(stream), launches)
        B.check(st, "padra_exl3_moe_decode_layer_launches")

    def moe_decode_layer_static(self, layer, ids, routing, normalized, x, tokens, stream=None):
        """The decode layer on the library's built-in scratch array: no workspace, no allocation in the call."""
        st = self.lib.padra_exl3_moe_decode_layer_static(self.t.descriptors.data_ptr(), layer, B.ptr(ids), B.ptr(routing),
                                                         B.ptr(normalized), B.ptr(x), tokens, self.t.rate, *self.dims,
                                                         B.ptr(self.table), B.ptr(self.bad), B.stream_handle(stream))
        B.check(st, "padra_exl3_moe_decode_layer_static")

    def moe_decode_layer(self, layer, ids, routing, normalized, x, tokens, stream=None):
        ws = self.decode_workspace(tokens)
        st = self.lib.padra_exl3_moe_decode_layer(self.t.descriptors.data_ptr(), layer, B.ptr(ids), B.ptr(routing),
                                                  B.ptr(normalized), B.ptr(x), tokens, self.t.rate, *self.dims,
                                                  B.ptr(self.table), B.ptr(ws), ws.numel(), B.ptr(self.bad),
                                                  B.stream_handle(stream))
        B.check(st, "padra_exl3_moe_decode_layer")

    def decode_weights(self, layer, expert, part, stream=None, tensor_form=False):
        """FP16 bit patterns [cols][rows] of one matrix through the kernels' codec (either of its two forms)."""
        rows, cols = self.t.shape(part)
        out = torch.empty((cols, rows), dtype=torch.uint16, device=self.t.device)
        entry = self.lib.padra_exl3_decode_weights_tensor if tensor_form else self.lib.padra_exl3_decode_weights
        st = entry(self.t.descriptor_ptr(layer, expert, part), B.ptr(out), rows, cols, self.t.rate, B.ptr(self.bad),
                   B.stream_handle(stream))
        B.check(st, "padra_exl3_decode_weights")
        return out

    def codec_ceiling(self, rate: int, form: int, iterations: int, blocks: int, stream=None) -> int:
        """Launches the register-only codec loop; returns the number of weights it decodes."""
        key = ("ceiling", blocks)
        if key not in self._workspace:
            self._workspace[key] = torch.empty(blocks * 256, dtype=torch.int32, device=self.t.device)
        st = self.lib.padra_codec_ceiling_launch(rate, form, iterations, blocks, B.ptr(self._workspace[key]), B.stream_handle(stream))
        B.check(st, "padra_codec_ceiling_launch")
        return blocks * 256 * 32 * iterations


# ---- synthetic inputs (seeded; shapes and distributions of the benchmark configurations) --------------------
def bf16_values(t: torch.Tensor) -> torch.Tensor:
    """FP32 tensor holding BF16-representable values (the decode-side activation convention)."""
    return t.to(torch.bfloat16).to(torch.float32)


def route_topk(logits: torch.Tensor):
    """Top-8 of 64 with softmax weights renormalised over the selection, BF16-valued, ascending expert id per
    token -- the layout the expert kernels expect from the router (reference: src/cuda/inference.cu:482-536).
    Used to synthesise routing for benchmarks; parity tests take routing from the CPU oracle instead."""
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, TOPK, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    ids, order = torch.sort(ids, dim=-1)
    w = torch.gather(w, -1, order)
    return ids.to(torch.int32).contiguous(), bf16_values(w).contiguous()


def zipf_logits(tokens: int, seed: int, s: float = 1.1, device="cuda", popularity_seed=None) -> torch.Tensor:
    """Router logits [tokens][64] (FP32) whose top-8 are distributed like zipf_routing's ids: log of the Zipf(s)
    popularity plus Gumbel noise (the eight largest of such sums are a sample without replacement with probability
    proportional to the popularity)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed if popularity_seed is None else popularity_seed)
    rank = torch.randperm(EXPERTS, generator=g)
    if popularity_seed is not None:
        g.manual_seed(seed)
    popularity = torch.empty(EXPERTS)
    popularity[rank] = torch.arange(1, EXPERTS + 1, dtype=torch.float32) ** (-s)
    u = torch.rand((tokens, EXPERTS), generator=g).clamp_(1e-9, 1 - 1e-9)
    return (popularity.log() - torch.log(-torch.log(u))).to(torch.float32).to(device).contiguous()


def zipf_routing(tokens: int, seed: int, s: float = 1.1, device="cuda", popularity_seed=None):
    """Routing with Zipf(s)-skewed expert popularity: per token, eight distinct experts sampled without
    replacement with probability proportional to rank^-s, the expert<->rank map a seeded permutation (seeded by
    `popularity_seed` when given, so that several chunks can share one popularity order)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed if popularity_seed is None else popularity_seed)
    rank = torch.randperm(EXPERTS, generator=g)
    if popularity_seed is not None:
        g.manual_seed(seed)
    popularity = torch.empty(EXPERTS)
    popularity[rank] = torch.arange(1, EXPERTS + 1, dtype=torch.float32) ** (-s)
    ids = torch.multinomial(popularity.expand(tokens, EXPERTS), TOPK, replacement=False, generator=g)
    ids, _ = torch.sort(ids, dim=-1)
    w = torch.rand((tokens, TOPK), generator=g) + 0.1
    w = w / w.sum(dim=-1, keepdim=True)
    return ids.to(torch.int32).to(device).contiguous(), bf16_values(w).to(device).contiguous()
