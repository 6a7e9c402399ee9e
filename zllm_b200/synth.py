"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no model file or dataset is involved).

Host-side numpy generators: the same bytes go to the CUDA kernels and to
whatever checks them, so "identical seeded inputs" is literal.
"""
from __future__ import annotations

import zlib

import numpy as np

Q8_0_BLOCK = (32, 34)    # elements, bytes (src/gguf/gguf.zig:79)
Q4_K_BLOCK = (256, 144)  # elements, bytes (src/ref/tensor.zig:100)


def rng_for(config: str, tensor: str) -> np.random.Generator:
    """One generator per (configuration, tensor name): seed = crc32 of both."""
    return np.random.default_rng(zlib.crc32(f"{config}/{tensor}".encode()))


def f16_uniform(rng: np.random.Generator, lo: float, hi: float, size) -> np.ndarray:
    """binary16 values uniform in [lo, hi] (as float16)."""
    return rng.uniform(lo, hi, size=size).astype(np.float16)


def q8_0_weights(rng: np.random.Generator, n: int, k: int, d_lo: float = 1e-4, d_hi: float = 2e-3,
                 signed_scales: bool = False) -> np.ndarray:
    """[n, k/32*34] uint8: blocks {f16 d, int8 q[32]}, q uniform in [-127, 127]."""
    assert k % 32 == 0
    nb = k // 32
    blocks = np.empty((n, nb, 34), dtype=np.uint8)
    q = rng.integers(-127, 128, size=(n, nb, 32), dtype=np.int8)
    blocks[:, :, 2:] = q.view(np.uint8)
    d = f16_uniform(rng, d_lo, d_hi, (n, nb))
    if signed_scales:
        d = d * rng.choice(np.array([-1, 1], dtype=np.float16), size=(n, nb))
    blocks[:, :, 0:2] = d.view(np.uint8).reshape(n, nb, 2)
    return blocks.reshape(n, nb * 34)


def q4_k_weights(rng: np.random.Generator, n: int, k: int, lo: float = 1e-4, hi: float = 1e-2,
                 signed_scales: bool = False) -> np.ndarray:
    """[n, k/256*144] uint8: super-blocks {f16 d, f16 dmin, scales[12], qs[128]}.

    Random bytes give nibbles uniform in 0..15 and, through the 6-bit packing
    of src/ref/tensor.zig:95-98, sub-block scales and mins uniform in 0..63.
    """
    assert k % 256 == 0
    nb = k // 256
    blocks = rng.integers(0, 256, size=(n, nb, 144), dtype=np.uint8)
    d = f16_uniform(rng, lo, hi, (n, nb, 2))
    if signed_scales:
        d = d * rng.choice(np.array([-1, 1], dtype=np.float16), size=(n, nb, 2))
    blocks[:, :, 0:4] = d.view(np.uint8).reshape(n, nb, 4)
    return blocks.reshape(n, nb * 144)


KQUANT_BLOCK_BYTES = {"q3_k": 110, "q5_k": 176, "q6_k": 210, "iq4_xs": 136}
_KQUANT_D_AT = {"q3_k": (108,), "q5_k": (0, 2), "q6_k": (208,), "iq4_xs": (0,)}   # byte offsets of the f16 super-scales


def kquant_weights(rng: np.random.Generator, ttype: str, n: int, k: int, lo: float = 1e-4, hi: float = 1e-2,
                   signed_scales: bool = False) -> np.ndarray:
    """[n, k/256 * block_bytes] uint8 in the GGUF file layout of Q3_K, Q5_K, Q6_K or IQ4_XS (src/ref/tensor.zig:54-181):
    random bytes for the packed values and sub-block scales, f16 super-scales uniform in [lo, hi]."""
    assert k % 256 == 0
    nb, bb = k // 256, KQUANT_BLOCK_BYTES[ttype]
    blocks = rng.integers(0, 256, size=(n, nb, bb), dtype=np.uint8)
    for at in _KQUANT_D_AT[ttype]:
        d = f16_uniform(rng, lo, hi, (n, nb, 1))
        if signed_scales:
            d = d * rng.choice(np.array([-1, 1], dtype=np.float16), size=(n, nb, 1))
        blocks[:, :, at:at + 2] = d.view(np.uint8).reshape(n, nb, 2)
    return blocks.reshape(n, nb * bb)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bits, round to nearest even (src/ref/matmul.zig:250-255)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = (b + (0x7FFF + ((b >> 16) & 1))) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def bf16_weights(rng: np.random.Generator, n: int, k: int, std: float = 0.02) -> np.ndarray:
    """[n, k] uint16 bf16 bits ~ N(0, std)."""
    return to_bf16_bits(rng.normal(0.0, std, size=(n, k)).astype(np.float32))


def normal_f32(rng: np.random.Generator, *shape, std: float = 1.0) -> np.ndarray:
    return rng.normal(0.0, std, size=shape).astype(np.float32)


def sigmoid(x: np.ndarray) -> np.ndarray:
    return (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)


def softplus(x: np.ndarray) -> np.ndarray:
    return np.log1p(np.exp(x.astype(np.float64))).astype(np.float32)


def deltanet_inputs(rng: np.random.Generator, tokens: int, k_heads: int, v_heads: int, d: int, bf16: bool = True):
    """Conv rows [q heads | k heads | v heads] with q, k L2-normalised per head
    (then rounded to bf16 when `bf16`), beta = sigmoid(N(0,1)), g = -softplus(N(0,1))."""
    q = normal_f32(rng, tokens, k_heads, d)
    k = normal_f32(rng, tokens, k_heads, d)
    v = normal_f32(rng, tokens, v_heads, d)
    if bf16:
        q, k, v = (bf16_bits_to_f32(to_bf16_bits(t)) for t in (q, k, v))
    q = q / np.sqrt((q.astype(np.float64) ** 2).sum(-1, keepdims=True)).astype(np.float32)
    k = k / np.sqrt((k.astype(np.float64) ** 2).sum(-1, keepdims=True)).astype(np.float32)
    if bf16:
        q, k = (bf16_bits_to_f32(to_bf16_bits(t)) for t in (q, k))
    conv = np.concatenate([q.reshape(tokens, -1), k.reshape(tokens, -1), v.reshape(tokens, -1)], axis=1)
    beta = sigmoid(normal_f32(rng, tokens, v_heads))
    g = -softplus(normal_f32(rng, tokens, v_heads))
    return np.ascontiguousarray(conv, dtype=np.float32), g, beta
