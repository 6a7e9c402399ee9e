"""Shared helpers of the parity tests."""
import numpy as np


def rel_err(got, want) -> float:
    """max|got - want| / max|want|: the reference's kernel-check metric (src/kernels/check.zig:212-222)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    scale = np.abs(want).max()
    return float(np.abs(got - want).max() / (scale if scale > 0 else 1.0))


def rel_l2(got, want) -> float:
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-300))


def bits(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def uniform(rng, shape, scale=1.0) -> np.ndarray:
    """Uniform in +-scale, as the reference's checks draw inputs (src/kernels/check.zig:133-137)."""
    return ((rng.random(shape, dtype=np.float32) * 2 - 1) * scale).astype(np.float32)


def split_q8_0(file_rows: np.ndarray, k: int) -> np.ndarray:
    """File-layout Q8_0 rows -> split rows (k int8, k/32 f16 scales, padded to 16 B): the layout
    repack_q8_0 produces (src/kernels/repack_q8_0.wgsl:1-5), built on the host to check the kernel."""
    n = file_rows.shape[0]
    blocks = file_rows.reshape(n, k // 32, 34)
    stride = (k + k // 16 + 15) & ~15
    out = np.zeros((n, stride), dtype=np.uint8)
    out[:, :k] = blocks[:, :, 2:].reshape(n, k)
    out[:, k:k + k // 16] = blocks[:, :, :2].reshape(n, k // 16)
    return out
