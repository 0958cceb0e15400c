"""Regenerates the golden vectors in this directory.

Decoder vectors come from the REFERENCE's own scalar decoder source (src/cuda/expert_exl3.cuh:4-22) compiled
for the host by oracle/Makefile into oracle/_ref/libref_weight.so, so this script needs the reference checkout
(make -C oracle ref).  The layer-arithmetic vectors come from the C oracle and pin it against regressions.
Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import exl3_oracle as O  # noqa: E402

OUT = Path(__file__).resolve().parent


def main():
    ref = O.RefWeight()
    co = O.COracle()
    rng = np.random.Generator(np.random.Philox(key=20261125))
    # 1. trellis decode, reference decoder: 32 outputs x 64 inputs per rate (8 tiles, incl. the cyclic wrap)
    for rate in (3, 4, 6):
        rows, cols = 32, 64
        data, _, _ = O.synthetic_matrix(rng, rows, cols, rate)
        w = ref.decode_matrix(data, rows, cols, rate)  # FP32 values of FP16 weights, [cols, rows]
        bits = w.astype(np.float16)
        assert (bits.astype(np.float32) == w).all()
        np.savez_compressed(OUT / f"decode_k{rate}.npz", data=data, rows=rows, cols=cols, rate=rate,
                            fp16_bits=bits.view(np.uint16))
    # 2. the codebook over every state, through the reference decoder: a K4 stream whose windows enumerate states
    #    is not constructible directly, so hash the oracle table and keep samples checked against the reference
    #    via one-tile streams: state s placed as the last 16 bits of tile position 255.
    table = O.mul1_bits(np.arange(65536, dtype=np.uint32))
    samples = np.arange(0, 65536, 61, dtype=np.uint32)
    sample_bits = np.empty(samples.size, dtype=np.uint16)
    perm = O.tile_permutation()
    i255, o255 = [int(v[0]) for v in np.where(perm == 255)]
    for n, s in enumerate(samples):
        words = np.zeros(32, dtype=np.uint32)  # K4 tile: position 255 ends at bit 1024 -> low 16 bits of word 31
        words[31] = s
        v = ref.lib.ref_weight(words.ctypes.data, 16, 16, 3, i255, o255)
        sample_bits[n] = np.float32(v).astype(np.float16).view(np.uint16)
    assert (sample_bits == table[samples]).all()
    np.savez_compressed(OUT / "mul1.npz", samples=samples, sample_bits=sample_bits,
                        table_sha256=np.frombuffer(hashlib.sha256(table.tobytes()).digest(), dtype=np.uint8))
    # 3. one K4 linear through the oracle (compensated form), plus SwiGLU table hash and routing cases
    rows, cols, rate = 128, 256, 4
    data, suh, svh = O.synthetic_matrix(rng, rows, cols, rate)
    x = O.bf16_round(rng.standard_normal(cols).astype(np.float32))
    m = co.matrix(data, suh, svh, rows, cols, rate)
    y, bad = co.linear(m, x)
    assert not bad
    silu = co.silu_table()
    logits = O.bf16_round(rng.standard_normal((4, 64)).astype(np.float32))
    ids, weights, bad = co.route(logits)
    assert not bad
    np.savez_compressed(OUT / "layer_math.npz", data=data, suh=suh, svh=svh, x=x, y=y, rows=rows, cols=cols, rate=rate,
                        silu_sha256=np.frombuffer(hashlib.sha256(silu.tobytes()).digest(), dtype=np.uint8),
                        silu_samples=silu[::257], logits=logits, route_ids=ids, route_weights=weights)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
