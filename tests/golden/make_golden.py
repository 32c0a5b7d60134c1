"""Generates the golden fixtures under tests/golden/ (run from the repository root:
``python tests/golden/make_golden.py``).

The reference stores no golden vectors and is Rust, so it cannot be imported or run
where these fixtures are made.  Each fixture is therefore computed here by an
INDEPENDENT route — pure-Python integers / numpy, never the C oracle or the CUDA
library — from the reference's own definitions:

  lcg.json        the hand-rolled recurrence that phobos-base/src/rng.rs:51-63 pins
                  Lcg against (seed 1, 2 and 42; raw states and unit floats as bit
                  patterns)
  masking.json    the exact-integer matmul of phobos-bench/examples/masking.rs:109-147
                  (A=(i%7)-3, B=(i%5)-2, 96x64x100): row checksums and corner values
  samples.json    the verifier's 64 xorshift sample positions for three extents
                  (phobos-bench/src/main.rs:403-416)
  f16.json        IEEE round-to-nearest-even f32->f16 on edge cases (numpy.float16;
                  the reference uses crate half 2.7.1, main.rs:447-449)
  flash.json      two-pass f64 softmax attention for a small seeded case (the
                  recurrence of main.rs:894-911 is mathematically the same function)
  tile.json       TileId packing (phobos-cluster/src/tile.rs:116-127) and arena size
                  classes (phobos-pod/src/tile_store.rs:228-242)
"""
import json
import struct
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
MASK = (1 << 64) - 1
A_, C_ = 6364136223846793005, 1442695040888963407


def lcg_states(seed, n):
    out, s = [], seed
    for _ in range(n):
        s = (s * A_ + C_) & MASK
        out.append(s)
    return out


def unit_bits(state):
    x = np.float32(state >> 33) / np.float32(1 << 31) - np.float32(1.0)
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def lcg_units(seed, n):
    return np.array([np.float32(s >> 33) / np.float32(1 << 31) - np.float32(1.0) for s in lcg_states(seed, n)],
                    dtype=np.float32)


def main():
    lcg = {}
    for seed in (1, 2, 42):
        st = lcg_states(seed, 16)
        lcg[str(seed)] = {"states": [str(s) for s in st], "unit_bits": [unit_bits(s) for s in st]}
    # element one million of stream 7 pins the skip-ahead
    s = 7
    for _ in range(1_000_000):
        s = (s * A_ + C_) & MASK
    lcg["skip"] = {"seed": 7, "index": 999_999, "state": str(s), "unit_bits": unit_bits(s)}
    (HERE / "lcg.json").write_text(json.dumps(lcg, indent=1))

    M, K, N = 96, 64, 100
    a = [[((i * K + k) % 7) - 3 for k in range(K)] for i in range(M)]
    b = [[((k * N + j) % 5) - 2 for j in range(N)] for k in range(K)]
    c = [[sum(a[i][k] * b[k][j] for k in range(K)) for j in range(N)] for i in range(M)]
    (HERE / "masking.json").write_text(json.dumps({
        "M": M, "K": K, "N": N, "row_sums": [sum(r) for r in c], "col_sums": [sum(c[i][j] for i in range(M)) for j in range(N)],
        "corners": [c[0][0], c[0][N - 1], c[M - 1][0], c[M - 1][N - 1]], "abs_sum": sum(abs(x) for r in c for x in r)}))

    def samples(rows, cols):
        state, out = 0x243F6A8885A308D3, []

        def nxt(limit):
            nonlocal state
            state ^= (state << 13) & MASK
            state ^= state >> 7
            state ^= (state << 17) & MASK
            return state % limit
        for s_ in range(64):
            if s_ == 0:
                out.append([0, 0])
            elif s_ == 1:
                out.append([rows - 1, cols - 1])
            else:
                i = nxt(rows)
                j = nxt(cols)
                out.append([i, j])
        return out
    (HERE / "samples.json").write_text(json.dumps({f"{r}x{c_}": samples(r, c_) for r, c_ in
                                                   ((4096, 4096), (8192, 8192), (4096, 64))}))

    edge = [0.0, -0.0, 1.0, -1.0, 65504.0, 65519.9, 65520.0, 65536.0, 1e-8, 2.0 ** -25, 2.0 ** -25 * 1.0000001,
            2.0 ** -24, 6.1e-5, 6.097555e-05, 0.1, 0.333333, 1.0009765625, 1.00048828125, 1.00146484375, 2049.0,
            2051.0, -3.14159, 1e6, -1e6, 5.9604645e-08, 3.0e-08]
    x = np.array(edge, dtype=np.float32)
    with np.errstate(over="ignore"):
        h = x.astype(np.float16)
    (HERE / "f16.json").write_text(json.dumps({"f32_bits": [int(v) for v in x.view(np.uint32)],
                                               "f16_bits": [int(v) for v in h.view(np.uint16)]}))

    Nq, Nk, D = 16, 48, 8
    q = lcg_units(11, Nq * D).astype(np.float16).astype(np.float64).reshape(Nq, D)
    k = lcg_units(12, Nk * D).astype(np.float16).astype(np.float64).reshape(Nk, D)
    v = lcg_units(13, Nk * D).astype(np.float16).astype(np.float64).reshape(Nk, D)
    s_ = q @ k.T * 0.35
    p = np.exp(s_ - s_.max(axis=1, keepdims=True))
    o = (p / p.sum(axis=1, keepdims=True)) @ v
    (HERE / "flash.json").write_text(json.dumps({"Nq": Nq, "Nk": Nk, "D": D, "scale": 0.35, "seeds": [11, 12, 13],
                                                 "out": [[float(x_) for x_ in r] for r in o]}))

    def tid(t, ver, coord):
        return (t << 52) | (ver << 36) | coord

    def size_class(b_):
        return max(256, -(-b_ // 256) * 256)
    (HERE / "tile.json").write_text(json.dumps({
        "ids": [[7, 3, 123456, str(tid(7, 3, 123456))], [4095, 65535, (1 << 36) - 1, str(tid(4095, 65535, (1 << 36) - 1))],
                [0, 0, 0, "0"], [1, 0, 5, str(tid(1, 0, 5))]],
        "size_class": [[0, 256], [1, 256], [256, 256], [257, 512], [10240 * 10240 * 4, size_class(10240 * 10240 * 4)]]}))
    print("wrote", sorted(p_.name for p_ in HERE.glob("*.json")))


if __name__ == "__main__":
    main()
