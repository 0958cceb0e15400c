"""Times the reference's own expert kernels (compiled unmodified for sm_100a into oracle/_ref/libref_kernels.so) beside
this library's, on the same GPU, the same weights and the same routing, at the only shape the reference's launchers
accept (hidden 2304, intermediate 896).  Run as `python -m tests.reference_kernel_timing` from the repository root on a
box where oracle/_ref was built; prints one JSON object.  Not collected by pytest (no test functions).

decode:  exl3_mma_dual::Launch(gate+up) + exl3_silu_lut::Activate + exl3_mma_dual::Launch(down) + Combine
         (src/cuda/inference.cu:2963-2975)  vs  padra_exl3_moe_decode_layer
prefill: fast_expert::Group + exl3_masked::Schedule + three exl3_transport_async64::Launch + packed Combine
         (src/cuda/inference.cu:3860-3921)  vs  the same sequence through padra_exl3_prefill_launch
"""
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def timed(fn, reps):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3  # microseconds


def main():
    from oracle import exl3_oracle as O
    from padra_b200 import binding as B
    from padra_b200.experts import ExpertKernels, ExpertTable, bf16_values, route_topk, zipf_routing

    gpu = torch.device("cuda:0")
    hidden, inter, rate, layers = 2304, 896, 4, 12  # 12 layers x 198 MB of weights rotate: larger than L2
    table = ExpertTable(layers, hidden, inter, rate, gpu).fill_random(7)
    k = ExpertKernels(table)
    ref = O.RefKernels()
    D, s = table.descriptors.data_ptr(), B.stream_handle()
    g = torch.Generator(device=gpu)
    g.manual_seed(3)
    bad = torch.zeros(1, dtype=torch.int32, device=gpu)
    out = {"shape": {"hidden": hidden, "inter": inter, "rate": rate, "layers_rotated": layers}}

    # ---- decode, one token ----
    ids, w = route_topk(bf16_values(torch.randn((1, 64), device=gpu, generator=g)))
    ids, w = ids.reshape(-1), w.reshape(-1)
    x = bf16_values(torch.randn((1, hidden), device=gpu, generator=g))
    rg, ru, rd = torch.zeros((8, inter), device=gpu), torch.zeros((8, inter), device=gpu), torch.zeros((8, hidden), device=gpu)
    rtable = torch.zeros(65536, dtype=torch.int16, device=gpu)
    ref.ref_silu_build(B.ptr(rtable), s)
    state = {"layer": 0}

    def reference_decode():
        layer = state["layer"] = (state["layer"] + 1) % layers
        rx = x.clone()
        ref.ref_decode_dual_launch(D, layer, 0, B.ptr(ids), B.ptr(x), B.ptr(rg), B.ptr(ru), 8, B.ptr(bad), s, rate)
        ref.ref_silu_activate(B.ptr(rg), B.ptr(ru), B.ptr(rtable), 8 * inter, B.ptr(bad), s)
        ref.ref_decode_dual_launch(D, layer, 2, B.ptr(ids), B.ptr(rg), B.ptr(rd), None, 8, B.ptr(bad), s, rate)
        ref.ref_combine(B.ptr(rx), B.ptr(rd), B.ptr(w), 1, B.ptr(bad), s)

    k.decode_workspace(1)

    def ours_decode():
        layer = state["layer"] = (state["layer"] + 1) % layers
        k.moe_decode_layer(layer, ids, w, x, x.clone(), 1)

    out["decode_1_token_us"] = {"reference_kernels": timed(reference_decode, 120), "this_library": timed(ours_decode, 120)}

    # ---- prefill, 2048 tokens, Zipf(1.1) ----
    tokens = 2048
    pairs = tokens * 8
    pids, pw = zipf_routing(tokens, seed=5, device=gpu)
    px = bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))
    groups = torch.zeros(64 * tokens, dtype=torch.int32, device=gpu)
    counts = torch.zeros(64, dtype=torch.int32, device=gpu)
    tiles = torch.zeros((pairs // 32 + 65, 3), dtype=torch.int32, device=gpu)
    tile_count = torch.zeros(1, dtype=torch.int32, device=gpu)
    rgate = torch.zeros((pairs, inter), dtype=torch.int16, device=gpu)
    rup = torch.zeros((pairs, inter), dtype=torch.int16, device=gpu)
    rdown = torch.zeros((pairs, hidden), dtype=torch.int16, device=gpu)
    work = torch.zeros((pairs, hidden), dtype=torch.float16, device=gpu)

    def reference_prefill():
        layer = state["layer"] = (state["layer"] + 1) % layers
        rx = px.clone()
        ref.ref_group(B.ptr(pids), B.ptr(groups), B.ptr(counts), tokens, B.ptr(bad), s)
        ref.ref_schedule(B.ptr(counts), B.ptr(tiles), B.ptr(tile_count), tokens, B.ptr(bad), s)
        for part, target in ((0, rgate), (1, rup), (2, rdown)):
            ref.ref_prefill_launch(D, layer, part, B.ptr(pids), B.ptr(groups), B.ptr(counts), B.ptr(tiles), B.ptr(tile_count),
                                   B.ptr(px), B.ptr(target), B.ptr(rgate), B.ptr(rup), B.ptr(k.table), B.ptr(work), tokens,
                                   B.ptr(bad), s, rate)
        ref.ref_combine_packed(B.ptr(rx), B.ptr(rdown), B.ptr(pw), tokens, B.ptr(bad), 1, s)

    def ours_prefill():
        layer = state["layer"] = (state["layer"] + 1) % layers
        k.prefill_layer(layer, pids.reshape(-1), pw.reshape(-1), px, px.clone(), tokens)

    out["prefill_2048_tokens_us"] = {"reference_kernels": timed(reference_prefill, 8), "this_library": timed(ours_prefill, 8)}
    assert int(bad.item()) == 0 and k.bad_flag() == 0
    for entry in ("decode_1_token_us", "prefill_2048_tokens_us"):
        out[entry]["speed_up"] = out[entry]["reference_kernels"] / out[entry]["this_library"]
    print(json.dumps(out))


if __name__ == "__main__":
    main()
