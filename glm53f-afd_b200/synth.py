"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The generator is the reference crate's SplitMix64 (crates/glm53f-kda/src/synth.rs:10-31) used counter-style:
value i of a stream is mix(state0 + (i+1) * gamma), so any slice of a stream can be produced independently and
the numpy code below yields exactly the sequence the reference's sequential `Rng` yields.  Normals come from
Box-Muller on two 24-bit uniforms, in double, rounded once to the storage type.

The distributions are those the benchmark configurations name: q, k, v ~ N(0,1) in bf16, q and k L2-normalised
per head (eps 1e-6 inside the root) and q scaled by 128^-0.5; per-channel log decay g = log(sigmoid(N(3,1)));
beta = sigmoid(N(0,1)); carried states ~ N(0, 0.05).
"""
from __future__ import annotations

import numpy as np

DK = DV = 128
_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_SEED_XOR = 0x6A09E667F3BCC909
_M64 = (1 << 64) - 1
BASE_SEED = 0x53454544


def stream_seed(config: int, layer: int, tag: str) -> int:
    """One stream per (configuration, layer, tensor tag)."""
    t = sum((i + 1) * b for i, b in enumerate(tag.encode())) & 0xFFFF
    return (BASE_SEED + config) ^ (layer << 20) ^ (t << 40)


def splitmix(seed: int, n: int, start: int = 0) -> np.ndarray:
    """Outputs start .. start+n-1 of the reference's `Rng::new(seed)` as uint64."""
    state0 = np.uint64((seed ^ _SEED_XOR) & _M64)
    idx = np.arange(start + 1, start + n + 1, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = state0 + idx * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform24(seed: int, n: int, start: int = 0) -> np.ndarray:
    """24-bit uniforms in [0, 1) as float64 (the reference's `uniform` before scaling)."""
    return (splitmix(seed, n, start) >> np.uint64(40)).astype(np.float64) / float(1 << 24)


def normal(seed: int, n: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    """N(mean, std) by Box-Muller: element i uses uniforms 2i and 2i+1 of the stream."""
    u = uniform24(seed, 2 * n)
    u1 = u[0::2] + 1.0 / float(1 << 24)  # (0, 1]
    u2 = u[1::2]
    return mean + std * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bits, round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def bf16_widen(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def sigmoid(x: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-x))


def tokens(config: int, layer: int, rows: int, heads: int):
    """q, k, v as bf16 bits [rows][H][128]; g f32 [rows][H][128]; beta f32 [rows][H]."""
    n = rows * heads * DK

    def unit(tag, scale):
        x = normal(stream_seed(config, layer, tag), n).astype(np.float32).reshape(rows * heads, DK)
        ss = np.sum(x * x, axis=1, keepdims=True, dtype=np.float32)
        x = x * (np.float32(1.0) / np.sqrt(ss + np.float32(1e-6)))
        return bf16_bits((x * np.float32(scale)).reshape(-1))

    q = unit("q", 1.0 / np.sqrt(128.0))
    k = unit("k", 1.0)
    v = bf16_bits(normal(stream_seed(config, layer, "v"), n).astype(np.float32))
    g = np.log(sigmoid(normal(stream_seed(config, layer, "g"), n, 3.0, 1.0))).astype(np.float32)
    beta = sigmoid(normal(stream_seed(config, layer, "beta"), rows * heads)).astype(np.float32)
    return q, k, v, g, beta


def state(config: int, layer: int, slot: int, heads: int, std: float = 0.05) -> np.ndarray:
    """A carried-over state N(0, std), f32 [H][128 (v)][128 (k)]."""
    return normal(stream_seed(config, layer, "state") ^ (slot << 8), heads * DV * DK, 0.0, std).astype(np.float32)


def varlen_lengths(config: int, total: int, lo: int = 256, hi: int = 2048) -> list[int]:
    """Sequence lengths uniform in [lo, hi], accepted until they sum to `total` (the last one clipped)."""
    out, used, i = [], 0, 0
    u = uniform24(stream_seed(config, 0, "lens"), 4 * (total // lo + 1))
    while used < total:
        n = min(lo + int(u[i] * (hi - lo + 1)), total - used)
        out.append(n)
        used += n
        i += 1
    return out
