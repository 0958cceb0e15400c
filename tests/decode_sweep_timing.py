"""configs[2]: rate and batch sweep of the decode layer call (K3, K4, K6 at M = 1, 2, 5, 16 tokens; M = 5 is an MTP D4
verify pass), and the prefill chunk at the three rates.  Run as `python -m tests.decode_sweep_timing` from the repository root; prints one JSON object with the
device time per layer step (CUDA graph of 28 steps over 28 layers of distinct weights, CUDA events) and the algorithmic
bytes per second.  Not collected by pytest (no test functions); parity of the same calls is in tests/test_gpu_decode.py."""
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    from padra_b200.experts import ExpertKernels, ExpertTable, bf16_values, route_topk

    gpu = torch.device("cuda:0")
    hidden, inter, layers = 2048, 1024, 28
    out = {"shape": {"hidden": hidden, "inter": inter, "layers_rotated": layers}, "results": []}
    g = torch.Generator(device=gpu)
    g.manual_seed(11)
    for rate in (3, 4, 6):
        table = ExpertTable(layers, hidden, inter, rate, gpu).fill_random(rate)
        k = ExpertKernels(table)
        for tokens in (1, 2, 5, 16):
            k.decode_workspace(tokens)
            steps = []
            for layer in range(layers):
                ids, w = route_topk(bf16_values(torch.randn((tokens, 64), device=gpu, generator=g)))
                steps.append((layer, ids.reshape(-1), w.reshape(-1), bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g)),
                              bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))))
            stream = torch.cuda.Stream(device=gpu)
            with torch.cuda.stream(stream):
                for s in steps[:3]:
                    k.moe_decode_layer(*s, tokens, stream=stream)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for s in steps:
                    k.moe_decode_layer(*s, tokens, stream=stream)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            a.record()
            for _ in range(reps):
                graph.replay()
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) / (reps * layers) * 1e3
            distinct = sum(len(torch.unique(s[1])) for s in steps) / layers
            nbytes = distinct * (3 * hidden * inter * rate // 8 + 6 * (hidden + inter)) + tokens * (hidden * 4 + 64)
            out["results"].append({"rate": rate, "tokens": tokens, "us_per_layer_step": us, "distinct_experts": distinct,
                                   "algorithmic_gb_per_s": nbytes / us / 1e3})
            assert k.bad_flag() == 0
        # the same weights through the prefill entry points: one 2048-token chunk per layer, Zipf(1.1) routing
        from padra_b200.experts import zipf_routing

        tokens = 2048
        chunks = []
        for layer in range(layers):
            ids, w = zipf_routing(tokens, seed=layer, device=gpu)
            chunks.append((layer, ids.reshape(-1), w.reshape(-1), bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g)),
                           bf16_values(torch.randn((tokens, hidden), device=gpu, generator=g))))
        for c in chunks[:3]:
            k.prefill_layer(*c, tokens)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for c in chunks:
            k.prefill_layer(*c, tokens)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / layers * 1e3
        out.setdefault("prefill_2048_tokens", []).append({"rate": rate, "us_per_layer_chunk": us,
                                                          "tflops": tokens * 8 * 3 * 2 * hidden * inter / us / 1e6})
        assert k.bad_flag() == 0
        del k, table
    print(json.dumps(out))


if __name__ == "__main__":
    main()
