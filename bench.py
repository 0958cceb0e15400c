"""Benchmark of the EXL3 MoE expert layer: decode (the headline), a prefill chunk, expert-parallel prefill.

Workload: one K4 MoE layer, hidden 2048, expert-intermediate 1024, 64 experts, top-8, ONE token per step.
A step is one pass of the whole expert layer (gate/up projections, SwiGLU, down projection, combine with
residual) through the library's C ABI.  Steps rotate over 28 layers of distinct synthetic weights (5.7 GB, far
larger than the 126 MB L2) so that every step streams its eight experts' packed weights from HBM.

Metric: achieved HBM GB/s over ALGORITHMIC bytes -- per step, the packed words and FP16 sidecars of the eight
selected experts' three matrices plus the token's activations and routing (25.3 MB at K4) -- divided by the
device time of the step.  `value` is measured with inputs resident in HBM (CUDA graphs, CUDA events);
`e2e` repeats the measurement through the same entry point with the step's inputs coming from pinned host
memory and its result read back, copies and synchronisation inside the timed region.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 (torchrun, one rank per GPU) every rank runs an independent replica of the decode workload (the
decode path does not shard); the value is the sum over ranks, timed as the maximum over ranks.

Two more objects ride on the same JSON line: `prefill_chunk` (N = 1: a 2048-token chunk, Zipf(1.1) routing, through
the tcgen05 grouped GEMM, with its tensor roofline) and `expert_parallel_prefill` (a 16384-token batch through all
layers with the experts sharded 64/N per GPU and the rows exchanged over NVLink peer memory; strong scaling).
`--impl reference` times the CPU restatement of the reference arithmetic (the reference has no CPU
implementation and no B200 build of this path) on the host cores, same metric and workload.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one gate+up SplitProjectionKernel launch, from the ncu capture
# summarised under profiles/ (16.88 MB read, nothing written back to DRAM inside the launch)
TRAFFIC_PER_LAUNCH = 16.88e6
WORKLOAD = "configs[1]: K4 MoE layer decode, 1 token, 64 experts top-8, hidden 2048, intermediate 1024"


def algorithmic_bytes(distinct_experts: int, tokens: int, hidden=HIDDEN, inter=INTER, rate=RATE) -> int:
    """Bytes a step must move: per distinct expert the packed words of three matrices and their FP16
    sidecars (suh and svh of each), plus per token the BF16 activation in and out and the routing entries."""
    per_expert = 3 * hidden * inter * rate // 8 + 2 * 2 * (hidden + inter) + 2 * (inter + hidden)
    return distinct_experts * per_expert + tokens * hidden * 2 * 2 + tokens * TOPK * 8


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
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
    steps, warmup = max(1, min(args.steps, 40)), max(1, min(args.warmup, 3))
    sec, nbytes = cpu_layer_steps(steps, warmup, threads)
    value = nbytes / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 x f16 -> f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "l2": "CPU arm; one layer's weights per step"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": f"{steps} whole layer steps (8 experts x 3 matrices, 25.3 MB packed each step) of the C "
                                   f"restatement of the reference arithmetic, OpenMP over outputs; the reference itself has no "
                                   f"CPU implementation of this path"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---- GPU arm ------------------------------------------------------------------------------------------------
def prefill_leg(k, dev, layers: int, tokens: int = 2048, passes: int = 3) -> dict:
    """One prefill chunk per layer (grouping, three grouped projections with the decode fused in, SwiGLU, combine) over
    `layers` layers of distinct weights, Zipf(1.1) routing; device time per chunk from CUDA events."""
    import torch
    from padra_b200.experts import bf16_values, zipf_routing

    g = torch.Generator(device=dev)
    g.manual_seed(77)
    chunks = []
    for layer in range(layers):
        ids, w = zipf_routing(tokens, seed=layer, device=dev)
        chunks.append((layer, ids.reshape(-1), w.reshape(-1), bf16_values(torch.randn((tokens, HIDDEN), device=dev, generator=g)),
                       bf16_values(torch.randn((tokens, HIDDEN), device=dev, generator=g))))
    for c in chunks[:3]:
        k.prefill_layer(*c, tokens)
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(passes):
        for c in chunks:
            k.prefill_layer(*c, tokens)
    b.record()
    torch.cuda.synchronize(dev)
    seconds = a.elapsed_time(b) / 1e3 / (passes * layers)
    flops = tokens * TOPK * 3 * 2 * HIDDEN * INTER
    measured = ROOT / "MEASURED_PEAKS.json"
    data = json.loads(measured.read_text()) if measured.exists() else {}
    tensor_peak = float(data.get("bf16_tflops_sustained", 1400.0))
    return {"workload": f"prefill chunk: {tokens} tokens x top-8 of 64 experts, hidden {HIDDEN} / inter {INTER}, K{RATE}, Zipf(1.1) routing",
            "tokens_per_s": tokens / seconds, "us_per_layer_chunk": seconds * 1e6, "tflops": flops / seconds / 1e12,
            "roofline": {"bound": "tensor", "achieved": flops / seconds / 1e12, "peak": tensor_peak, "unit": "TFLOP/s",
                         "frac": flops / seconds / 1e12 / tensor_peak,
                         "peak_source": "measured (sustained cuBLAS bf16)" if data else "fallback"},
            "kernels_per_chunk": 9, "layers_rotated": layers, "passes": passes}


def expert_parallel_leg(k, dev, world: int, rank: int, layers: int, exchange: str, batch: int = 16384, chunk: int = 2048) -> dict:
    """configs[4]: a batch of 16384 tokens through `layers` MoE layers, experts sharded 64/world per rank by measured
    popularity, tokens split evenly over the ranks (strong scaling), all-to-all dispatch and combine per layer and
    chunk.  Between layers the next input is the RMS-normalised residual stream, so layer l+1 depends on layer l.
    Returns this rank's device time; the caller takes the maximum over ranks."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from padra_b200 import expert_parallel as EP
    from padra_b200.experts import bf16_values, zipf_routing

    local = batch // world
    if world > 1 and exchange == "nccl" and local <= chunk:
        chunk = local // 2  # at least two chunks per rank, so that exchange and expert work overlap
    chunks = [(c, min(chunk, local - c)) for c in range(0, local, chunk)]
    g = torch.Generator(device=dev)
    g.manual_seed(500 + rank)
    x0 = bf16_values(torch.randn((local, HIDDEN), device=dev, generator=g))
    routing, owners = {}, []
    for layer in range(layers):
        # popularity as a server would have measured it over earlier traffic: a long sample of the layer's routing
        sample, _ = zipf_routing(16384, seed=layer, device="cpu", popularity_seed=layer)
        popularity = np.bincount(sample.reshape(-1).numpy(), minlength=EXPERTS)
        owners.append(EP.balanced_placement(popularity, world))
        for c, n in chunks:
            ids, w = zipf_routing(n, seed=10007 * layer + (rank * local + c) // chunk + 1, device=dev, popularity_seed=layer)
            routing[layer, c] = (ids.reshape(-1), w.reshape(-1))
    engines = peer = None
    if world > 1 and exchange == "nccl":
        backend, group_exchange = EP.KernelBackend(k), EP.GroupExchange()
        engines = [EP.ExpertParallelPrefill(backend, group_exchange, owners[layer]) for layer in range(layers)]
    elif world > 1:
        # symmetric memory may be unavailable on a host (no peer access, no handle exchange): every rank then takes the
        # NCCL exchange, and the JSON line says which exchange ran
        try:
            peer = EP.PeerExchangePrefill.over_group(k, owners[0], cap=chunk * TOPK)
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

    def normalise(rows):  # stand-in for the model's RMSNorm between layers (outside the measured path's scope)
        return torch.nn.functional.rms_norm(rows, (HIDDEN,), eps=1e-6).to(torch.bfloat16).float()

    def stack(x):
        for layer in range(layers):
            if peer is not None:  # rows stored straight into the owners' memory over NVLink, nothing returns to the host
                for c, n in chunks:
                    rows = x[c:c + n]
                    peer.layer(layer, *routing[layer, c], normalise(rows), rows, owner=device_owners[layer])
            elif engines is None:
                for c, n in chunks:
                    rows = x[c:c + n]
                    k.prefill_layer(layer, *routing[layer, c], normalise(rows), rows, n)
            else:  # NCCL all-to-all, all of the layer's chunks in one pipelined call
                engines[layer].layer_chunks(layer, [(*routing[layer, c], normalise(x[c:c + n]), x[c:c + n]) for c, n in chunks])

    stack(x0.clone())  # warm-up: workspaces, NCCL channels
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    x = x0.clone()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    stack(x)
    b.record()
    torch.cuda.synchronize(dev)
    assert k.bad_flag() == 0 and bool(torch.isfinite(x).all()), "expert-parallel prefill raised the error flag"
    return {"seconds": a.elapsed_time(b) / 1e3, "batch": batch, "layers": layers, "chunk": chunk, "exchange": exchange}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable, bf16_values, route_topk

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
    table = ExpertTable(layers, HIDDEN, INTER, RATE, dev).fill_random(seed=rank)
    k = ExpertKernels(table)
    variants = 2
    g = torch.Generator(device=dev)
    g.manual_seed(1000 + rank)
    slots = []
    for v in range(variants):
        for layer in range(layers):
            ids, w = route_topk(bf16_values(torch.randn((TOKENS, EXPERTS), device=dev, generator=g)))
            normalized = bf16_values(torch.randn((TOKENS, HIDDEN), device=dev, generator=g))
            x = bf16_values(torch.randn((TOKENS, HIDDEN), device=dev, generator=g))
            slots.append({"layer": layer, "ids": ids.reshape(-1), "w": w.reshape(-1), "normalized": normalized, "x": x})
    k.decode_workspace(TOKENS)
    stream = torch.cuda.Stream(device=dev)
    bytes_per_step = algorithmic_bytes(TOPK, TOKENS)

    def layer_call(s, st):
        k.moe_decode_layer(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], TOKENS, stream=st)

    # one CUDA graph per (layer, routing variant): the step as a serving loop would replay it
    with torch.cuda.stream(stream):
        for s in slots[:2]:
            layer_call(s, stream)
    stream.synchronize()
    kernels_per_step = 2  # split-K gate+up projection and split-K down projection, each with its epilogue inside
    for s in slots:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                layer_call(s, stream)
        s["graph"] = graph

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(steps, fn):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            start.record(stream)
            for i in range(steps):
                fn(i)
            stop.record(stream)
        stop.synchronize()
        barrier()
        return start.elapsed_time(stop) / 1e3

    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            slots[i % len(slots)]["graph"].replay()
    with ClockSampler(local) as clocks:
        seconds = timed(args.steps, lambda i: slots[i % len(slots)]["graph"].replay())
        # the dominant kernel alone (gate+up split-K projection: 16.0 MiB of the step's 24 MiB of packed words): a CUDA
        # graph of one such launch per layer, so that the GPU and not the launching thread sets the pace; CUDA events
        # on the launching stream around whole replays, divided by the launches they contain
        kernel_graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(kernel_graph, stream=stream):
                for s in slots[:layers]:
                    k.moe_decode_layer_launches(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], TOKENS, 1, stream=stream)
            for _ in range(3):
                kernel_graph.replay()
            ev_a, ev_b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            kernel_reps = max(3, min(args.steps, 560) // layers)
            ev_a.record(stream)
            for _ in range(kernel_reps):
                kernel_graph.replay()
            ev_b.record(stream)
        ev_b.synchronize()
        kernel_ms = [ev_a.elapsed_time(ev_b) / (kernel_reps * layers)]
        # for comparison: the same layer as the reference's call sequence of separate launches (per-part entry points)
        unfused_graphs = []
        for s in slots[:min(len(slots), 28)]:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                k.moe_decode_layer_unfused(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], TOKENS, stream=stream)
                stream.synchronize()
                with torch.cuda.graph(graph, stream=stream):
                    k.moe_decode_layer_unfused(s["layer"], s["ids"], s["w"], s["normalized"], s["x"], TOKENS, stream=stream)
            unfused_graphs.append(graph)
        unfused_steps = min(args.steps, 280)
        unfused_seconds = timed(unfused_steps, lambda i: unfused_graphs[i % len(unfused_graphs)].replay())
    clock_info = clocks.summary()
    assert k.bad_flag() == 0, "the sticky error flag was raised during the benchmark"

    # end to end: the step's inputs start in pinned host memory, its result is read back, every step
    host = []
    for s in slots:
        host.append({n: s[n].cpu().pin_memory() for n in ("ids", "w", "normalized", "x")})
    result = torch.empty((TOKENS, HIDDEN), dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host[0].values())
    d2h = result.numel() * result.element_size()

    # the whole step as a serving loop would replay it: copies in, the layer call, copy out, one graph per slot
    # (the copies are graph nodes that read and write the pinned host buffers on every replay)
    for s, h in zip(slots, host):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                for n in ("ids", "w", "normalized", "x"):
                    s[n].copy_(h[n], non_blocking=True)
                layer_call(s, stream)
                result.copy_(s["x"], non_blocking=True)
        s["e2e_graph"] = graph

    def e2e_step(i):
        slots[i % len(slots)]["e2e_graph"].replay()
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

    ep = expert_parallel_leg(k, dev, world, rank, layers, args.ep_exchange) if EXPERTS % world == 0 and not args.no_ep else None
    if world > 1:
        t = torch.tensor([seconds, e2e_seconds, ep["seconds"] if ep else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds, e2e_seconds = float(t[0]), float(t[1])
        if ep:
            ep["seconds"] = float(t[2])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    total_bytes = bytes_per_step * args.steps * world
    value = total_bytes / seconds / 1e9
    peak, peak_source = peaks()
    kernel_s = statistics.mean(kernel_ms) / 1e3
    # gate+up launch: packed words and suh of 8 experts x 2 matrices, the token row, the FP32 slice sums it writes
    kernel_bytes = TOPK * 2 * (HIDDEN * INTER * RATE // 8 + 2 * HIDDEN) + TOKENS * HIDDEN * 4 + TOPK * 2 * 4 * INTER * 4
    achieved = kernel_bytes / kernel_s / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": seconds / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 x f16 -> f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rate": RATE, "layers_rotated": layers, "weight_bytes_resident": table.total_bytes,
                   "l2": f"inputs larger than L2: {layers} layers x 203 MB of expert weights rotate, 126 MB L2",
                   "bytes_per_step": bytes_per_step, "multi_gpu": "independent replicas (decode does not shard)"},
        "frac_of_hbm_peak": value / world / peak,
        "roofline": {"bound": "hbm", "kernel": "LayerProjectionKernel<4,1,0>, gate+up launch (dominant kernel of the step)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_source,
                     "bytes_per_launch": kernel_bytes, "us_per_launch": kernel_s * 1e6, "traffic": TRAFFIC_PER_LAUNCH},
        "unfused_call_sequence": {"value": bytes_per_step * unfused_steps / unfused_seconds / 1e9, "unit": "GB/s",
                                  "ms_per_step": unfused_seconds / unfused_steps * 1e3, "kernels_per_step": 4},
        "e2e": {"value": total_bytes / e2e_seconds / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_seconds / args.steps * 1e3},
        "gpu_launches": kernels_per_step * args.steps,
        "clocks": {"sm_mhz": clock_info["sm_mhz"], "sm_max_mhz": clock_info["sm_max_mhz"], "reasons": clock_info["reasons"],
                   "samples": clock_info["samples"]},
    }
    if ep:
        flops = ep["batch"] * TOPK * 3 * 2 * HIDDEN * INTER * ep["layers"]
        line["expert_parallel_prefill"] = {
            "workload": f"configs[4]: {ep['batch']}-token batch through {ep['layers']} K{RATE} MoE layers, experts sharded 64/{world} per GPU "
                        "by measured popularity, Zipf(1.1) routing, dispatch and return " +
                        ("by kernels storing into peer memory over NVLink (symmetric memory, epoch flags)" if ep["exchange"] == "peer"
                         else "by NCCL all-to-all, chunks pipelined over two streams") if world > 1 else
                        f"configs[4] at one GPU: {ep['batch']}-token batch through {ep['layers']} K{RATE} MoE layers in chunks of {ep['chunk']}",
            "n_gpus": world, "scaling": "strong", "tokens_per_s": ep["batch"] / ep["seconds"], "ms_per_batch": ep["seconds"] * 1e3,
            "tflops_all_gpus": flops / ep["seconds"] / 1e12, "timing": "CUDA events on each rank, maximum over ranks"}
    if world == 1:
        line["prefill_chunk"] = prefill_leg(k, dev, layers)
        assert k.bad_flag() == 0, "the sticky error flag was raised during the prefill leg"
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
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel exchange: kernels over NVLink peer memory (default) or NCCL all-to-all")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layers of distinct weights to rotate over (profiling: fewer)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
