"""Benchmark of the EXL3 MoE expert layer: decode (the headline), a prefill chunk, expert-parallel prefill.

Workload: one K4 MoE layer, hidden 2048, expert-intermediate 1024, 64 experts, top-8, ONE token per step.
A step is one pass of the whole expert layer (gate/up projections, SwiGLU, down projection, combine with
residual) through the library's C ABI.  Steps rotate over 28 layers of distinct synthetic weights (5.7 GB, far
larger than the 126 MB L2) so that every step streams its eight experts' packed weights from HBM.

Metric: achieved HBM GB/s over ALGORITHMIC bytes -- per step, the packed words and FP16 sidecars of the eight
selected experts' three matrices plus the token's activations and routing (25.3 MB at K4) -- divided by the
device time of the step.  `value` is measured with inputs resident in HBM (CUDA graphs of 28 consecutive layer
steps, CUDA events); `e2e` repeats the measurement through the same entry point with every step's inputs coming
from pinned host memory and its result read back, copies and synchronisation inside the timed region.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 (torchrun, one rank per GPU) every rank runs an independent replica of the decode workload (the
decode path does not shard); the value is the sum over ranks, timed as the maximum over ranks.

More objects ride on the same JSON line.  At every N: `expert_parallel_prefill` (configs[4]: a 16384-token batch
through all layers with the experts sharded 64/N per GPU and the rows exchanged over NVLink peer memory; strong
scaling; checked against the single-GPU path before it is timed).  At N = 1: `roofline_issue` (the codec's
instruction-issue ceiling, measured), `decode_sweep` (configs[2]: K3/K4/K6 at 1, 2, 5, 16 tokens), `prefill_chunk`
(configs[3]), `reference_kernels_b200` (the reference's own kernels compiled for this GPU, where that library was
built) and `cpu_baseline`.  `--impl reference` times the CPU restatement of the reference arithmetic (the
reference has no CPU implementation and no B200 build of this path) on the host cores, same metric and workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, INTER, EXPERTS, TOPK, RATE, LAYERS, TOKENS = 2048, 1024, 64, 8, 4, 28, 1
METRIC = "exl3_k4_moe_layer_decode_hbm_gbs"
# DRAM bytes (read + written) of one launch of the dominant kernel, the gate+up projection, measured with ncu
TRAFFIC_PER_LAUNCH = 16.92e6
WORKLOAD = "configs[1]: K4 MoE layer decode, 1 token, 64 experts top-8, hidden 2048, intermediate 1024"
MIN_TIMED_SECONDS = 0.05


def base_config(layers: int) -> dict:
    """The keys both arms print, so that the two lines describe the same workload."""
    return {"workload": WORKLOAD, "rate": RATE, "hidden": HIDDEN, "inter": INTER, "experts": EXPERTS, "top_k": TOPK, "tokens": TOKENS,
            "layers_rotated": layers, "bytes_per_step": algorithmic_bytes(TOPK, TOKENS)}


def algorithmic_bytes(distinct_experts: float, tokens: int, hidden=HIDDEN, inter=INTER, rate=RATE) -> float:
    """Bytes a step must move: per distinct expert the packed words of three matrices and their FP16
    sidecars (suh and svh of each), plus per token the BF16 activation in and out and the routing entries."""
    per_expert = 3 * hidden * inter * rate // 8 + 2 * 2 * (hidden + inter) + 2 * (inter + hidden)
    return distinct_experts * per_expert + tokens * hidden * 2 * 2 + tokens * TOPK * 8


def measured_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text()) if p.exists() else {}


def hbm_peak():
    data = measured_peaks()
    if "hbm_gbs" in data:
        return float(data["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.file = index, None, None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()  # the exact child started above
            self.proc.wait(timeout=10)

    def summary(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.file is None:
            return out
        self.file.flush()
        rows = [r.split(",") for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 7]
        os.unlink(self.file.name)
        sm, reasons = [], set()
        for r in rows:
            try:
                sm.append(float(r[0]))
                out["sm_max_mhz"] = float(r[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            out["sm_mhz"] = statistics.median(sm)
        out["reasons"], out["samples"] = sorted(reasons), len(sm)
        return out


# ---- CPU arm ------------------------------------------------------------------------------------------------
def cpu_layer_steps(steps: int, warmup: int, threads: int):
    """Times `steps` layer steps of the CPU restatement (all three projections of eight experts, SwiGLU,
    combine) with `threads` OpenMP threads.  Returns (seconds per step, bytes per step)."""
    import numpy as np

    from oracle import exl3_oracle as O

    co = O.COracle()
    co.lib.exl3_set_threads(threads)
    rng = np.random.Generator(np.random.Philox(key=0))
    mats = (O.Matrix * (EXPERTS * 3))()
    keep = []
    x = O.bf16_round(rng.standard_normal((1, HIDDEN)).astype(np.float32))
    ids, w, _ = co.route(O.bf16_round(rng.standard_normal((1, EXPERTS)).astype(np.float32)))
    for e in ids.reshape(-1):  # only the selected experts need host weights
        for part in range(3):
            rows, cols = (HIDDEN, INTER) if part == 2 else (INTER, HIDDEN)
            data, suh, svh = O.synthetic_matrix(rng, rows, cols, RATE)
            keep.append((data, suh, svh))
            m = mats[int(e) * 3 + part]
            m.data, m.suh, m.svh = data.ctypes.data, suh.ctypes.data, svh.ctypes.data
            m.rows, m.cols, m.format = rows, cols, O.FORMAT_OF_RATE[RATE]
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        out, bad = co.moe_layer(mats, 0, ids, w, x, HIDDEN, INTER, f16_form=True)
        dt = time.perf_counter() - t0
        assert not bad
        if i >= warmup:
            times.append(dt)
    return sum(times) / len(times), algorithmic_bytes(TOPK, TOKENS)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU arm runs once per box
    threads = os.cpu_count() or 1
    # a bounded sample: the CPU needs about 0.1 s per step, so at most 60 timed steps and at most the warm-up asked for
    steps, warmup = max(1, min(args.steps, 60)), max(0, min(args.warmup, 8))
    sec, nbytes = cpu_layer_steps(steps, warmup, threads)
    value = nbytes / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 x f16 -> f32", "data": "synthetic", "config": base_config(args.layers),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{steps} timed whole layer steps after {warmup} warm-up steps (8 experts x 3 matrices, 25.3 MB packed "
                                   f"each step) of the C restatement of the reference arithmetic, OpenMP over outputs; the reference "
                                   f"itself has no CPU implementation of this path"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---- GPU arm: helpers ---------------------------------------------------------------------------------------
def decode_slots(table_layers, tokens, dev, generator, variants=2, hidden=HIDDEN):
    """Inputs of `variants` x layers decode steps: fresh routing, normalised input and residual row(s) each."""
    import torch
    from padra_b200.experts import bf16_values, route_topk

    slots = []
    for _ in range(variants):
        for layer in range(table_layers):
            ids, w = route_topk(bf16_values(torch.randn((tokens, EXPERTS), device=dev, generator=generator)))
            fields = {"ids": ids.reshape(-1), "w": w.reshape(-1),
                      "normalized": bf16_values(torch.randn((tokens, hidden), device=dev, generator=generator)),
                      "x": bf16_values(torch.randn((tokens, hidden), device=dev, generator=generator))}
            # the step's inputs sit back to back in ONE device buffer (256-byte aligned fields), so that a host that holds
            # them the same way brings them over with one copy
            offsets, total = {}, 0
            for name, t in fields.items():
                offsets[name] = total
                total += (t.numel() * t.element_size() + 255) // 256 * 256
            packed = torch.zeros(total, dtype=torch.uint8, device=dev)
            slot = {"layer": layer, "packed": packed}
            for name, t in fields.items():
                view = packed[offsets[name]:offsets[name] + t.numel() * t.element_size()].view(t.dtype).view(t.shape)
                view.copy_(t)
                slot[name] = view
            slots.append(slot)
    return slots


def capture(stream, fn):
    """One CUDA graph of whatever fn enqueues on `stream` (run once uncaptured first: lazy set-up happens there)."""
    import torch

    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
    return graph


def time_replays(stream, graphs, repeats):
    """Seconds per pass over `graphs`, CUDA events on the launching stream, after three warm-up passes."""
    import torch

    with torch.cuda.stream(stream):
        for _ in range(3):
            for g in graphs:
                g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(repeats):
            for g in graphs:
                g.replay()
        b.record(stream)
    b.synchronize()
    return a.elapsed_time(b) / 1e3 / repeats


def decode_sweep_leg(dev, layers: int) -> list:
    """configs[2]: K3 / K4 / K6 packed weights at 1, 2, 5 and 16 tokens, routing drawn per token from seeded N(0,1) logits;
    the layer call over `layers` layers of distinct weights in one CUDA graph."""
    import torch
    from padra_b200.experts import ExpertKernels, ExpertTable

    out = []
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    stream = torch.cuda.Stream(device=dev)
    for rate in (3, 4, 6):
        table = ExpertTable(layers, HIDDEN, INTER, rate, dev).fill_random(rate)
        k = ExpertKernels(table)
        for tokens in (1, 2, 5, 16):
            k.decode_workspace(tokens)
            slots = decode_slots(layers, tokens, dev, g, variants=1)
            graph = capture(stream, lambda: [k.moe_decode_layer(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], tokens, stream=stream)
                                             for s in slots])
            seconds = time_replays(stream, [graph], 8) / layers
            distinct = sum(len(torch.unique(s["ids"])) for s in slots) / layers
            nbytes = algorithmic_bytes(distinct, tokens, rate=rate)
            out.append({"rate": rate, "tokens": tokens, "distinct_experts": round(distinct, 1), "us_per_step": round(seconds * 1e6, 2),
                        "gbs": round(nbytes / seconds / 1e9, 1)})
            assert k.bad_flag() == 0, "the sticky error flag was raised during the rate and batch sweep"
        del k, table
        torch.cuda.empty_cache()
    return out


def prefill_leg(k, dev, layers: int, tokens: int = 2048, passes: int = 3) -> dict:
    """configs[3]: one prefill chunk per layer (routing from Zipf(1.1)-skewed logits, grouping, the grouped projections with the
    decode fused in, SwiGLU, combine) over `layers` layers of distinct weights; device time per chunk from CUDA events."""
    import torch
    from padra_b200.experts import bf16_values, zipf_logits

    g = torch.Generator(device=dev)
    g.manual_seed(77)
    chunks = []
    for layer in range(layers):
        chunks.append((layer, zipf_logits(tokens, seed=layer, device=dev), bf16_values(torch.randn((tokens, HIDDEN), device=dev, generator=g)),
                       bf16_values(torch.randn((tokens, HIDDEN), device=dev, generator=g))))
    for c in chunks[:3]:
        k.prefill_chunk(*c, tokens)
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(passes):
        for c in chunks:
            k.prefill_chunk(*c, tokens)
    b.record()
    torch.cuda.synchronize(dev)
    seconds = a.elapsed_time(b) / 1e3 / (passes * layers)
    flops = tokens * TOPK * 3 * 2 * HIDDEN * INTER
    data = measured_peaks()
    burst, sustained = float(data.get("bf16_tflops", 1590.0)), float(data.get("bf16_tflops_sustained", 1400.0))
    achieved = flops / seconds / 1e12
    return {"workload": f"configs[3]: {tokens} tokens x top-8 of 64 experts, hidden {HIDDEN} / inter {INTER}, K{RATE}, Zipf(1.1) routing",
            "tokens_per_s": tokens / seconds, "us_per_layer_chunk": seconds * 1e6, "tflops": achieved,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst,
                         "frac_of_sustained": achieved / sustained,
                         "peak_source": "measured (cuBLAS bf16 burst; the chunk is well under a second)" if data else "fallback"},
            "launches_per_chunk": 6,
            "chunk": "router logits -> residual stream: routing + grouping + schedule, gate+up input transform, gate+up grouped GEMM, "
                     "down input transform (SwiGLU), down grouped GEMM, combine",
            "layers_rotated": layers, "passes": passes}


def reference_kernels_leg(dev) -> dict | None:
    """The reference's own kernels, compiled unmodified for this GPU (oracle/_ref/libref_kernels.so, built where the reference
    checkout is present), timed beside this library at the only shape the reference's launchers accept (2304 / 896)."""
    import torch
    from oracle import exl3_oracle as O

    if not O.RefKernels.available():
        return None
    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable, bf16_values, route_topk, zipf_routing

    hidden, inter, rate, layers = 2304, 896, 4, 12  # 12 layers x 198 MB of weights rotate: larger than L2
    table = ExpertTable(layers, hidden, inter, rate, dev).fill_random(7)
    k = ExpertKernels(table)
    ref = O.RefKernels()
    D, s = table.descriptors.data_ptr(), B.stream_handle()
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    state = {"layer": 0}

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize(dev)
        return a.elapsed_time(b) / reps * 1e3

    ids, w = route_topk(bf16_values(torch.randn((1, 64), device=dev, generator=g)))
    ids, w = ids.reshape(-1), w.reshape(-1)
    x = bf16_values(torch.randn((1, hidden), device=dev, generator=g))
    rg, ru, rd = torch.zeros((8, inter), device=dev), torch.zeros((8, inter), device=dev), torch.zeros((8, hidden), device=dev)
    rtable = torch.zeros(65536, dtype=torch.int16, device=dev)
    ref.ref_silu_build(B.ptr(rtable), s)
    rx, ox = x.clone(), x.clone()

    def reference_decode():  # src/cuda/inference.cu:2963-2975
        layer = state["layer"] = (state["layer"] + 1) % layers
        ref.ref_decode_dual_launch(D, layer, 0, B.ptr(ids), B.ptr(x), B.ptr(rg), B.ptr(ru), 8, B.ptr(bad), s, rate)
        ref.ref_silu_activate(B.ptr(rg), B.ptr(ru), B.ptr(rtable), 8 * inter, B.ptr(bad), s)
        ref.ref_decode_dual_launch(D, layer, 2, B.ptr(ids), B.ptr(rg), B.ptr(rd), None, 8, B.ptr(bad), s, rate)
        ref.ref_combine(B.ptr(rx), B.ptr(rd), B.ptr(w), 1, B.ptr(bad), s)

    k.decode_workspace(1)

    def ours_decode():
        layer = state["layer"] = (state["layer"] + 1) % layers
        k.moe_decode_layer(layer, ids, w, x, ox, 1)

    out = {"shape": {"hidden": hidden, "inter": inter, "rate": rate, "layers_rotated": layers},
           "decode_1_token_us": {"reference_kernels": timed(reference_decode, 120), "this_library": timed(ours_decode, 120)}}
    tokens = 2048
    pairs = tokens * 8
    pids, pw = zipf_routing(tokens, seed=5, device=dev)
    px = bf16_values(torch.randn((tokens, hidden), device=dev, generator=g))
    groups = torch.zeros(64 * tokens, dtype=torch.int32, device=dev)
    counts = torch.zeros(64, dtype=torch.int32, device=dev)
    tiles = torch.zeros((pairs // 32 + 65, 3), dtype=torch.int32, device=dev)
    tile_count = torch.zeros(1, dtype=torch.int32, device=dev)
    rgate, rup = (torch.zeros((pairs, inter), dtype=torch.int16, device=dev) for _ in range(2))
    rdown = torch.zeros((pairs, hidden), dtype=torch.int16, device=dev)
    work = torch.zeros((pairs, hidden), dtype=torch.float16, device=dev)
    prx, pox = px.clone(), px.clone()

    def reference_prefill():  # src/cuda/inference.cu:3860-3921
        layer = state["layer"] = (state["layer"] + 1) % layers
        ref.ref_group(B.ptr(pids), B.ptr(groups), B.ptr(counts), tokens, B.ptr(bad), s)
        ref.ref_schedule(B.ptr(counts), B.ptr(tiles), B.ptr(tile_count), tokens, B.ptr(bad), s)
        for part, target in ((0, rgate), (1, rup), (2, rdown)):
            ref.ref_prefill_launch(D, layer, part, B.ptr(pids), B.ptr(groups), B.ptr(counts), B.ptr(tiles), B.ptr(tile_count),
                                   B.ptr(px), B.ptr(target), B.ptr(rgate), B.ptr(rup), B.ptr(k.table), B.ptr(work), tokens,
                                   B.ptr(bad), s, rate)
        ref.ref_combine_packed(B.ptr(prx), B.ptr(rdown), B.ptr(pw), tokens, B.ptr(bad), 1, s)

    def ours_prefill():
        layer = state["layer"] = (state["layer"] + 1) % layers
        k.prefill_layer(layer, pids.reshape(-1), pw.reshape(-1), px, pox, tokens)

    out["prefill_2048_tokens_us"] = {"reference_kernels": timed(reference_prefill, 8), "this_library": timed(ours_prefill, 8)}
    for entry in ("decode_1_token_us", "prefill_2048_tokens_us"):
        out[entry]["speed_up"] = out[entry]["reference_kernels"] / out[entry]["this_library"]
    # both sides run unchecked residual streams for many steps here (values grow without a norm in between): the flags are not read
    return out


def expert_parallel_leg(k, dev, world: int, rank: int, layers: int, exchange: str, passes: int, batch: int = 16384,
                        chunk: int = 2048, replicas: int = 1, engine_count: int = 2, returns: str = "auto") -> dict:
    """configs[4]: a batch of 16384 tokens through `layers` MoE layers, experts sharded 64/world per rank by measured
    popularity, tokens split evenly over the ranks (strong scaling), dispatch and combine per layer and chunk.  Between
    layers the next input is the RMS-normalised residual stream (this library's norm kernel), so layer l+1 depends on
    layer l.  Before anything is timed, one chunk of one layer goes through the exchange path AND through the single-GPU
    prefill path on the same tokens, and the two results must be equal bit for bit on every rank.
    Returns this rank's device times; the caller takes the maximum over ranks."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from padra_b200 import expert_parallel as EP
    from padra_b200.experts import bf16_values, zipf_routing

    local = batch // world
    if world > 1:  # at least one chunk per engine, so that one chunk's exchange overlaps the others' expert work
        chunk = min(chunk, max(256, local // engine_count))
    chunks = [(c, min(chunk, local - c)) for c in range(0, local, chunk)]
    if returns == "auto":  # two halves pay for their extra launches on 2048-token chunks (40.1 against 40.5 ms on four GPUs), not on
        returns = "split" if chunk >= 2048 else "plain"  # 1024-token chunks (22.3 against 22.0 ms on eight)
    g = torch.Generator(device=dev)
    g.manual_seed(500 + rank)
    x0 = bf16_values(torch.randn((local, HIDDEN), device=dev, generator=g))
    norm_weight = torch.full((HIDDEN,), 0x3F80, dtype=torch.int16, device=dev)  # BF16 ones
    routing, owners, loads = {}, [], []
    for layer in range(layers):
        # popularity as a server would have measured it over earlier traffic: a long sample of the layer's routing
        sample, _ = zipf_routing(16384, seed=layer, device="cpu", popularity_seed=layer)
        popularity = np.bincount(sample.reshape(-1).numpy(), minlength=EXPERTS)
        owners.append(EP.balanced_placement(popularity, world, replicas=abs(replicas), force=replicas < 0))
        loads.append((EP.placement_load(popularity, EP.balanced_placement(popularity, world), world),
                      EP.placement_load(popularity, owners[-1], world)))
        for c, n in chunks:
            ids, w = zipf_routing(n, seed=10007 * layer + (rank * local + c) // chunk + 1, device=dev, popularity_seed=layer)
            routing[layer, c] = (ids.reshape(-1), w.reshape(-1))
    engines = peer = device_owners = None
    if world > 1 and exchange == "nccl":
        backend, group_exchange = EP.KernelBackend(k), EP.GroupExchange()
        engines = [EP.ExpertParallelPrefill(backend, group_exchange, owners[layer]) for layer in range(layers)]
    elif world > 1:
        # symmetric memory may be unavailable on a host (no peer access, no handle exchange): every rank then takes the
        # NCCL exchange, and the JSON line says which exchange ran
        try:  # engines with an exchange block each: the chunks of a layer go to them in turn, on a stream each
            peer = [EP.PeerExchangePrefill.over_group(k, owners[0], cap=chunk * TOPK, fused_return=returns == "fused",
                                                      split_return=returns == "split") for _ in range(engine_count)]
            failed = 0
        except Exception as error:  # noqa: BLE001 - any failure of the rendezvous means "not available here"
            print(f"rank {rank}: peer exchange unavailable ({type(error).__name__}: {error}); using NCCL all-to-all", file=sys.stderr)
            peer, failed = None, 1
        vote = torch.tensor([failed], device=dev)
        dist.all_reduce(vote, op=dist.ReduceOp.MAX)
        if int(vote.item()):
            peer, exchange = None, "nccl"
            backend, group_exchange = EP.KernelBackend(k), EP.GroupExchange()
            engines = [EP.ExpertParallelPrefill(backend, group_exchange, owners[layer]) for layer in range(layers)]
        else:
            device_owners = [torch.from_numpy(o.astype(np.int32)).to(dev) for o in owners]
    lanes = engine_count if peer is not None else 1
    normalized = [torch.empty((chunk, HIDDEN), dtype=torch.float32, device=dev) for _ in range(lanes)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(lanes)] if peer is not None else None

    def normalise(rows, lane=0):  # the post-attention norm's place: this library's kernel, weight of ones
        out = normalized[lane][:rows.shape[0]]
        k.residual_norm(rows, None, out, norm_weight)
        return out

    def one_layer(layer, c, n, x, lane=0):
        rows = x[c:c + n]
        if peer is not None:  # rows stored straight into the owners' memory over NVLink, nothing returns to the host
            peer[lane].layer(layer, *routing[layer, c], normalise(rows, lane), rows, owner=device_owners[layer])
        elif engines is None:
            k.prefill_layer(layer, *routing[layer, c], normalise(rows), rows, n)
        else:
            engines[layer].layer(layer, *routing[layer, c], normalise(rows), rows)

    def stack(x):
        main = torch.cuda.current_stream()
        for layer in range(layers):
            if engines is not None:  # NCCL all-to-all, all of the layer's chunks in one pipelined call
                pieces = []
                for c, n in chunks:
                    rows = x[c:c + n]
                    pieces.append((*routing[layer, c], normalise(rows).clone(), rows))
                engines[layer].layer_chunks(layer, pieces)
            elif peer is not None:
                # the layer's chunks alternate between the two engines; the layer ends when both streams have finished
                # (every token of layer l+1 waits for layer l of the whole rank, as it would behind an attention block)
                start = torch.cuda.Event()
                start.record(main)
                for lane, stream in enumerate(streams):
                    stream.wait_event(start)
                    with torch.cuda.stream(stream):
                        for c, n in chunks[lane::lanes]:
                            one_layer(layer, c, n, x, lane)
                    done = torch.cuda.Event()
                    done.record(stream)
                    main.wait_event(done)
            else:
                for c, n in chunks:
                    one_layer(layer, c, n, x)

    # ---- parity of the exchange path against the single-GPU path, same tokens, same weights (every rank holds all of them) ----
    parity_rows = 0
    if world > 1:
        c, n = chunks[0]
        through_exchange, alone = x0.clone(), x0.clone()
        one_layer(0, c, n, through_exchange)
        k.prefill_layer(0, *routing[0, c], normalise(alone[c:c + n]).clone(), alone[c:c + n], n)
        torch.cuda.synchronize(dev)
        equal = torch.equal(through_exchange[c:c + n], alone[c:c + n]) and k.bad_flag() == 0
        verdict = torch.tensor([0 if equal else 1], device=dev)
        dist.all_reduce(verdict, op=dist.ReduceOp.MAX)
        assert int(verdict.item()) == 0, f"rank {rank}: the {exchange} exchange path differs from the single-GPU prefill path"
        assert not torch.equal(alone[c:c + n], x0[c:c + n]), "the parity check compared untouched rows"
        parity_rows = n

    stack(x0.clone())  # warm-up: workspaces, NCCL channels
    torch.cuda.synchronize(dev)
    times = []
    for _ in range(passes):
        if world > 1:
            dist.barrier()
        x = x0.clone()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        stack(x)
        b.record()
        torch.cuda.synchronize(dev)
        times.append(a.elapsed_time(b) / 1e3)
        assert k.bad_flag() == 0 and bool(torch.isfinite(x).all()), "expert-parallel prefill raised the error flag"
    return {"times": times, "batch": batch, "layers": layers, "chunk": chunk, "exchange": exchange, "parity_rows": parity_rows,
            "engines": lanes, "returns": returns,
            "placement": {"layers_with_a_second_copy_of_the_hottest_expert": int(sum(bool((np.asarray(o) >> 8).any()) for o in owners)),
                          "busiest_rank_over_mean_64_per_rank_exact": round(float(np.mean([a for a, _ in loads])), 4),
                          "busiest_rank_over_mean_as_run": round(float(np.mean([b for _, b in loads])), 4)}}


# ---- GPU arm ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = B.load()
    assert lib.padra_device_supported() == B.OK, "not an sm_100 device"

    layers = args.layers
    table = ExpertTable(layers, HIDDEN, INTER, RATE, dev).fill_random(seed=0)  # the same weights on every rank
    k = ExpertKernels(table)
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    slots = decode_slots(layers, TOKENS, dev, g, variants=2)
    k.decode_workspace(TOKENS)
    stream = torch.cuda.Stream(device=dev)
    bytes_per_step = algorithmic_bytes(TOPK, TOKENS)

    def layer_call(s):
        k.moe_decode_layer(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], TOKENS, stream=stream)

    # The step as a serving loop replays it: CUDA graphs.  One graph holds `layers` consecutive layer steps (the expert
    # layers of one token's pass through the model, each with routing and inputs of its own); a graph of the first few
    # layers covers what is left when the step count is not a multiple of the layer count.
    passes = [capture(stream, lambda v=v: [layer_call(s) for s in slots[v * layers:(v + 1) * layers]]) for v in range(2)]
    partial = {}
    kernels_per_step = 2  # split-K gate+up projection; split-K down projection with the gate/up epilogue in front and the combine behind

    def run_steps(count):
        full, rest = divmod(count, layers)
        for i in range(full):
            passes[i % 2].replay()
        if rest:
            partial[rest].replay()

    for rest in {args.warmup % layers, args.steps % layers} - {0}:  # captured here, outside every timed region
        partial[rest] = capture(stream, lambda rest=rest: [layer_call(s) for s in slots[:rest]])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed_steps(count):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            start.record(stream)
            run_steps(count)
            stop.record(stream)
        stop.synchronize()
        barrier()
        return start.elapsed_time(stop) / 1e3

    with torch.cuda.stream(stream):
        run_steps(args.warmup)
    with ClockSampler(local) as clocks:
        # exactly `steps` steps per timed region; the region is repeated until at least 50 ms have been timed, and the
        # median region is reported
        regions = [timed_steps(args.steps)]
        while sum(regions) < MIN_TIMED_SECONDS and len(regions) < 400:
            regions.append(timed_steps(args.steps))
        seconds = statistics.median(regions)
        # the dominant kernel alone (gate+up split-K projection: 16.0 MiB of the step's 24 MiB of packed words): a CUDA
        # graph of one such launch per layer, so that the GPU and not the launching thread sets the pace
        kernel_graph = capture(stream, lambda: [k.moe_decode_layer_launches(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], TOKENS, 1,
                                                                             stream=stream) for s in slots[:layers]])
        kernel_s = time_replays(stream, [kernel_graph], max(3, min(args.steps, 560) // layers)) / layers
        # for comparison: the same layer as the reference's call sequence of separate launches (per-part entry points)
        unfused = capture(stream, lambda: [k.moe_decode_layer_unfused(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], TOKENS,
                                                                       stream=stream) for s in slots[:layers]])
        unfused_s = time_replays(stream, [unfused], max(3, min(args.steps, 280) // layers)) / layers
    clock_info = clocks.summary()
    assert k.bad_flag() == 0, "the sticky error flag was raised during the benchmark"

    # end to end: the step's inputs start in pinned host memory, its result is read back, every step; one graph per step
    # (copies in, the layer call, copy out) replayed and synchronised, as a serving loop does per token and layer
    host = [s["packed"].cpu().pin_memory() for s in slots]
    result = torch.empty((TOKENS, HIDDEN), dtype=torch.float32).pin_memory()
    h2d = host[0].numel() * host[0].element_size()
    d2h = result.numel() * result.element_size()

    def e2e_graph(s, h):
        def enqueue():
            s["packed"].copy_(h, non_blocking=True)  # ids, routing weights, normalised input, residual row: one copy
            layer_call(s)
            result.copy_(s["x"], non_blocking=True)
        return capture(stream, enqueue)

    e2e_graphs = [e2e_graph(s, h) for s, h in zip(slots, host)]

    def e2e_step(i):
        e2e_graphs[i % len(e2e_graphs)].replay()
        stream.synchronize()

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        for i in range(args.steps):
            e2e_step(i)
    torch.cuda.synchronize(dev)
    e2e_seconds = time.perf_counter() - t0
    barrier()

    ep = None
    if EXPERTS % world == 0 and not args.no_ep:
        if world > 1 and args.ep_exchange == "peer":  # leave SMs to the other engine's exchange kernels beside the persistent GEMM
            B.check(k.lib.padra_prefill_set_reserved_sms(args.ep_reserved_sms), "padra_prefill_set_reserved_sms")
        ep = expert_parallel_leg(k, dev, world, rank, layers, args.ep_exchange, passes=args.ep_passes, replicas=args.ep_replicas,
                                 engine_count=args.ep_engines, returns=args.ep_return)
        B.check(k.lib.padra_prefill_set_reserved_sms(0), "padra_prefill_set_reserved_sms")
    if world > 1:
        t = torch.tensor([seconds, e2e_seconds] + (ep["times"] if ep else []), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds, e2e_seconds = float(t[0]), float(t[1])
        if ep:
            ep["times"] = [float(v) for v in t[2:]]
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    total_bytes = bytes_per_step * args.steps * world
    value = total_bytes / seconds / 1e9
    peak, peak_source = hbm_peak()
    # gate+up launch: packed words and suh of 8 experts x 2 matrices, the token row, the FP32 slice sums it writes
    kernel_bytes = TOPK * 2 * (HIDDEN * INTER * RATE // 8 + 2 * HIDDEN) + TOKENS * HIDDEN * 4 + TOPK * 2 * 4 * INTER * 4
    achieved = kernel_bytes / kernel_s / 1e9
    line = {"metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 x f16 -> f32", "data": "synthetic"}
    if ep:
        flops = ep["batch"] * TOPK * 3 * 2 * HIDDEN * INTER * ep["layers"]
        best = statistics.median(ep["times"])
        line["expert_parallel_prefill"] = {
            "workload": f"configs[4]: {ep['batch']} tokens x {ep['layers']} K{RATE} MoE layers, experts 64/{world} per GPU",
            "n_gpus": world, "scaling": "strong", "exchange": ep["exchange"] if world > 1 else "none", "ms_per_batch": best * 1e3,
            "ms_per_batch_min": min(ep["times"]) * 1e3, "passes": len(ep["times"]), "tokens_per_s": ep["batch"] / best,
            "tflops_all_gpus": flops / best / 1e12, "parity_checked": world > 1, "parity_rows": ep["parity_rows"],
            "placement": ep["placement"], "chunk_tokens": ep["chunk"], "engines": ep["engines"], "return_mode": ep["returns"],
            "timing": "CUDA events per rank, max over ranks, median of passes"}
    line.update({
        "config": dict(base_config(layers), weight_bytes_resident=table.total_bytes,
                       l2=f"inputs larger than L2: {layers} layers x 203 MB of expert weights rotate, 126 MB L2",
                       graph=f"{layers} consecutive layer steps per CUDA graph",
                       timed_regions=len(regions), multi_gpu="independent replicas (decode does not shard)"),
        "frac_of_hbm_peak": value / world / peak,
        "roofline": {"bound": "hbm", "kernel": "SingleGateUpKernel<4>, the gate+up launch (dominant kernel of the step)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_source,
                     "bytes_per_launch": kernel_bytes, "us_per_launch": kernel_s * 1e6, "traffic": TRAFFIC_PER_LAUNCH},
        "e2e": {"value": total_bytes / e2e_seconds / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_seconds / args.steps * 1e3},
        "gpu_launches": kernels_per_step * args.steps,
        "clocks": {"sm_mhz": clock_info["sm_mhz"], "sm_max_mhz": clock_info["sm_max_mhz"], "reasons": clock_info["reasons"],
                   "samples": clock_info["samples"]},
        "unfused_call_sequence": {"value": bytes_per_step / unfused_s / 1e9, "unit": "GB/s", "ms_per_step": unfused_s * 1e3,
                                  "kernels_per_step": 4},
    })
    if world == 1 and not args.quick:
        # the codec's instruction-issue ceiling: its inner loop on registers alone, with the FP16 mma attached (what the decode
        # kernels execute per weight), all SMs, eight CTAs of 256 threads each
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        best = 0.0
        for _ in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                k.codec_ceiling(RATE, 2, 200, sms * 8, stream)
                a.record(stream)
                weights = k.codec_ceiling(RATE, 2, 2000, sms * 8, stream)
                b.record(stream)
            b.synchronize()
            best = max(best, weights / (a.elapsed_time(b) / 1e3))
        weights_per_step = TOPK * 3 * HIDDEN * INTER
        line["roofline_issue"] = {"what": "trellis decode + FP16 mma on registers alone (no memory traffic), K4", "unit": "weights/s",
                                  "ceiling_weights_per_s": best, "achieved": weights_per_step / (seconds / args.steps),
                                  "frac": weights_per_step / (seconds / args.steps) / best,
                                  "step_us_at_ceiling": weights_per_step / best * 1e6,
                                  "gbs_at_ceiling": bytes_per_step / (weights_per_step / best) / 1e9}
        line["prefill_chunk"] = prefill_leg(k, dev, layers)
        assert k.bad_flag() == 0, "the sticky error flag was raised during the prefill leg"
        line["decode_sweep"] = decode_sweep_leg(dev, layers)
        reference_kernels = reference_kernels_leg(dev)
        if reference_kernels:
            line["reference_kernels_b200"] = reference_kernels
    if world == 1 and not args.no_cpu:
        threads = os.cpu_count() or 1
        sec, nbytes = cpu_layer_steps(steps=12, warmup=1, threads=threads)
        line["cpu_baseline"] = {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": "12 whole layer steps of the same workload (8 experts x 3 matrices per step) through "
                                          "the C restatement of the reference arithmetic, OpenMP over outputs"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=560)
    ap.add_argument("--warmup", type=int, default=56)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-ep", action="store_true", help="skip the expert-parallel prefill leg")
    ap.add_argument("--quick", action="store_true", help="headline only: skip the ceiling, sweep, prefill and reference-kernel legs")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel exchange: kernels over NVLink peer memory (default) or NCCL all-to-all")
    ap.add_argument("--ep-passes", type=int, default=5, help="timed passes of the expert-parallel batch (median reported)")
    ap.add_argument("--ep-replicas", type=int, default=2,
                    help="k > 0: up to k of a layer's most popular experts are held by two ranks, as long as that lowers the "
                         "busiest rank's load; -k: held by two ranks in any case (exercises the path on two or four GPUs)")
    ap.add_argument("--ep-reserved-sms", type=int, default=0, help="SMs the grouped GEMM leaves free for the exchange kernels (several GPUs)")
    ap.add_argument("--ep-return", default="auto", choices=["auto", "split", "fused", "plain"],
                    help="how the down rows travel back: in two halves beside the second half's GEMM, from the GEMM's epilogue, "
                         "or by one kernel after the GEMM")
    ap.add_argument("--ep-engines", type=int, default=2, help="exchange engines (blocks and streams) per rank that take a layer's chunks in turn")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers of distinct weights to rotate over (profiling: fewer)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
