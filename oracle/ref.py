"""ctypes binding of the CPU oracle (oracle/ref_cpu.cpp).

TEST INFRASTRUCTURE, NOT PRODUCT CODE: only tests/, the smoke check and the
bench's CPU-baseline leg import this module. The CUDA path never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"

# GGUF tensor type ids (src/gguf/gguf.zig TensorType).
F32, F16, Q8_0, Q3_K, Q4_K, Q5_K, Q6_K, IQ4_XS, BF16 = 0, 1, 8, 11, 12, 13, 14, 23, 30
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q8_0: (32, 34), Q4_K: (256, 144), Q3_K: (256, 110), Q5_K: (256, 176),
         Q6_K: (256, 210), IQ4_XS: (256, 136)}

# Accumulation modes of ref_matmul / ref_delta_rule.
MUL_ADD, FMA, F64 = 0, 1, 2


def build() -> None:
    """Compiles the three ISA flavours (a no-op when they are up to date)."""
    subprocess.run(["make", "-C", str(HERE), "-s"], check=True)


def _cpu_flags() -> set[str]:
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def _pick() -> Path:
    flags = _cpu_flags()
    want = []
    if {"avx512f", "avx512vl", "avx512bw", "avx512dq", "avx2", "fma", "f16c"} <= flags:
        want.append("libref_cpu_avx512.so")
    if {"avx2", "fma", "f16c"} <= flags:
        want.append("libref_cpu_avx2.so")
    want.append("libref_cpu.so")
    for name in want:
        if (BUILD / name).exists():
            return BUILD / name
    build()
    for name in want:
        if (BUILD / name).exists():
            return BUILD / name
    raise RuntimeError("oracle library missing; run `make -C oracle`")


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    L = C.CDLL(str(_pick()))
    f32p, u8p, u16p, vp, sz = C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.POINTER(C.c_uint16), C.c_void_p, C.c_size_t
    sig = {
        "ref_f16_to_f32": (C.c_float, [C.c_uint16]),
        "ref_f32_to_f16": (C.c_uint16, [C.c_float]),
        "ref_dequantize": (C.c_int, [C.c_int, vp, vp, sz]),
        "ref_dot": (C.c_float, [vp, vp, sz]),
        "ref_rms_norm": (None, [vp, vp, sz, C.c_float]),
        "ref_l2_norm": (None, [vp, sz, C.c_float]),
        "ref_silu": (C.c_float, [C.c_float]),
        "ref_sigmoid": (C.c_float, [C.c_float]),
        "ref_softplus": (C.c_float, [C.c_float]),
        "ref_rope_cos_sin": (None, [C.c_uint32, sz, sz, C.c_float, C.c_float, vp]),
        "ref_rope": (None, [vp, C.c_uint32, sz, C.c_float]),
        "ref_rope_normal": (None, [vp, C.c_uint32, sz, C.c_float, vp]),
        "ref_rope_table": (None, [vp, sz, sz, C.c_float, vp]),
        "ref_softmax": (None, [vp, sz]),
        "ref_round_like_llama": (None, [C.c_int, vp, sz]),
        "ref_pool_create": (vp, [sz]),
        "ref_pool_destroy": (None, [vp]),
        "ref_pool_threads": (sz, [vp]),
        "ref_matrix_create": (vp, [vp, C.c_int, vp, sz, sz]),
        "ref_matrix_destroy": (None, [vp]),
        "ref_matrix_row": (None, [vp, sz, vp]),
        "ref_matmul": (None, [vp, vp, vp, vp, sz, C.c_int, C.c_int]),
        "ref_attend_decode": (None, [vp, vp, vp, sz, vp, vp, sz, sz, sz, sz, C.c_float, vp, sz]),
        "ref_conv_norm": (None, [vp, vp, vp, sz, sz, sz, sz, sz, C.c_float]),
        "ref_delta_rule": (None, [vp, vp, vp, vp, vp, vp, sz, sz, sz, sz, C.c_int]),
        "ref_gated_norm": (None, [vp, vp, vp, sz, sz, sz, C.c_float]),
        "ref_dense_decode_layer": (None, [vp, vp, vp, vp, vp, C.c_uint32, sz, sz, sz, sz, sz, C.c_float, C.c_float, C.c_float, C.c_int]),
        "ref_dense_head": (None, [vp, vp, vp, vp, vp, sz, C.c_float, C.c_int]),
        "ref_build_info": (C.c_char_p, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def physical_cores() -> int:
    """Threads the reference would use: one per physical core (src/main.zig:438-448)."""
    try:
        seen = set()
        phys = core = None
        for line in open("/proc/cpuinfo"):
            if line.startswith("physical id"):
                phys = line.split(":")[1].strip()
            elif line.startswith("core id"):
                core = line.split(":")[1].strip()
            elif not line.strip():
                if phys is not None and core is not None:
                    seen.add((phys, core))
                phys = core = None
        if seen:
            return min(len(seen), len(os.sched_getaffinity(0)))
    except OSError:
        pass
    return max(1, len(os.sched_getaffinity(0)))


class Pool:
    def __init__(self, threads: int | None = None):
        self.h = lib().ref_pool_create(threads or physical_cores())

    @property
    def threads(self) -> int:
        return lib().ref_pool_threads(self.h)

    def close(self):
        if self.h:
            lib().ref_pool_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()


_default_pool = None


def default_pool() -> Pool:
    global _default_pool
    if _default_pool is None:
        _default_pool = Pool()
    return _default_pool


def dequantize(ttype: int, data: np.ndarray, n: int) -> np.ndarray:
    """ref/tensor.zig:21-43."""
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    if lib().ref_dequantize(ttype, _p(data), _p(out), n) != 0:
        raise ValueError("UnsupportedTensorType")
    return out


def round_like_llama(ttype: int, x) -> np.ndarray:
    x = _f32(x).copy()
    lib().ref_round_like_llama(ttype, _p(x), x.size)
    return x


def f16_round(x) -> np.ndarray:
    """KvFormat.f16.round (ref/qwen35.zig:32-42)."""
    return round_like_llama(F16, x)


def to_f16_bits(x) -> np.ndarray:
    x = _f32(x)
    f = lib().ref_f32_to_f16
    return np.array([f(float(v)) for v in x.ravel()], dtype=np.uint16).reshape(x.shape) if x.size < 4096 else _f16_bits_fast(x)


def _f16_bits_fast(x: np.ndarray) -> np.ndarray:
    # numpy's float32 -> float16 cast is IEEE round-to-nearest-even as well; the
    # small-size path above pins it against the oracle's own converter in tests.
    return x.astype(np.float16).view(np.uint16)


def rms_norm(x, w, eps: float) -> np.ndarray:
    x = _f32(x).copy()
    w = _f32(w)
    lib().ref_rms_norm(_p(x), _p(w), x.size, eps)
    return x


def l2_norm(x, eps: float) -> np.ndarray:
    x = _f32(x).copy()
    lib().ref_l2_norm(_p(x), x.size, eps)
    return x


def rope(x, pos: int, n_rot: int, base: float) -> np.ndarray:
    x = _f32(x).copy()
    lib().ref_rope(_p(x), pos, n_rot, base)
    return x


def rope_normal(x, pos: int, n_rot: int, base: float, factors=None) -> np.ndarray:
    x = _f32(x).copy()
    f = None if factors is None else _f32(factors)
    lib().ref_rope_normal(_p(x), pos, n_rot, base, _p(f))
    return x


def rope_table(positions: int, n_rot: int, base: float, factors=None) -> np.ndarray:
    t = np.empty(positions * (n_rot // 2) * 2, dtype=np.float32)
    f = None if factors is None else _f32(factors)
    lib().ref_rope_table(_p(t), positions, n_rot, base, _p(f))
    return t


def softmax(x) -> np.ndarray:
    x = _f32(x).copy()
    lib().ref_softmax(_p(x), x.size)
    return x


def dot(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().ref_dot(_p(a), _p(b), a.size)


class Matrix:
    """ref/matmul.zig:37-107: an n x k weight matrix of a GGUF type."""

    def __init__(self, ttype: int, data: np.ndarray, n: int, k: int, pool: Pool | None = None):
        be, bb = BLOCK[ttype]
        self.bytes = np.ascontiguousarray(data).view(np.uint8).ravel()
        assert self.bytes.size == n * k // be * bb, (self.bytes.size, n, k)
        self.n, self.k, self.type = n, k, ttype
        self.pool = pool or default_pool()
        self.h = lib().ref_matrix_create(self.pool.h, ttype, _p(self.bytes), n, k)
        if not self.h:
            raise ValueError("UnsupportedTensorType")

    def row(self, j: int) -> np.ndarray:
        out = np.empty(self.k, dtype=np.float32)
        lib().ref_matrix_row(self.h, j, _p(out))
        return out

    def dense(self) -> np.ndarray:
        """All rows decoded to f32 (n x k)."""
        if BLOCK[self.type][0] > 1:
            return dequantize(self.type, self.bytes, self.n * self.k).reshape(self.n, self.k)
        return np.stack([self.row(j) for j in range(self.n)])

    def __del__(self):
        if getattr(self, "h", None):
            lib().ref_matrix_destroy(self.h)
            self.h = None


def matmul(x, w: Matrix, act: bool = False, mode: int = MUL_ADD, pool: Pool | None = None) -> np.ndarray:
    """ref/matmul.zig:160-195: out[t][j] = sum_i x[t][i] * w[j][i]."""
    x = _f32(x).reshape(-1, w.k)
    rows = x.shape[0]
    out = np.empty((rows, w.n), dtype=np.float32)
    lib().ref_matmul((pool or w.pool).h, _p(out), _p(x), w.h, rows, int(act), mode)
    return out


def attend_decode(q, kc_bits, vc_bits, keys: int, heads: int, kv_heads: int, hd: int, scale: float,
                  gate=None, pool: Pool | None = None) -> np.ndarray:
    """ref/dense.zig:252-274 for one query at position keys-1; q is [heads, hd]."""
    q = _f32(q).reshape(heads, hd)
    kc = np.ascontiguousarray(kc_bits, dtype=np.uint16)
    vc = np.ascontiguousarray(vc_bits, dtype=np.uint16)
    out = np.empty((heads, hd), dtype=np.float32)
    g = None if gate is None else _f32(gate).reshape(heads, hd)
    lib().ref_attend_decode((pool or default_pool()).h, _p(out), _p(q), hd, _p(kc), _p(vc), keys, heads, kv_heads, hd,
                            scale, _p(g), hd)
    return out


def conv_norm(qkv, taps_w, n: int, k_heads: int, inner: int, d: int, kernel: int, eps: float) -> np.ndarray:
    qkv, taps_w = _f32(qkv), _f32(taps_w)
    out = np.empty_like(qkv)
    lib().ref_conv_norm(_p(out), _p(qkv), _p(taps_w), n, k_heads, inner, d, kernel, eps)
    return out


def delta_rule(state, conv, g, beta, n: int, k_heads: int, v_heads: int, d: int, mode: int = MUL_ADD,
               pool: Pool | None = None):
    """ref/qwen35.zig:493-546 before the norm/gate. Returns (new_state, out[n, v_heads*d])."""
    state = _f32(state).copy()
    conv, g, beta = _f32(conv), _f32(g), _f32(beta)
    out = np.empty((n, v_heads * d), dtype=np.float32)
    lib().ref_delta_rule((pool or default_pool()).h, _p(state), _p(out), _p(conv), _p(g), _p(beta), n, k_heads,
                         v_heads, d, mode)
    return state, out


def gated_norm(o, z, norm_w, n: int, v_heads: int, d: int, eps: float) -> np.ndarray:
    o = _f32(o).copy()
    z, norm_w = _f32(z), _f32(norm_w)
    lib().ref_gated_norm(_p(o), _p(z), _p(norm_w), n, v_heads, d, eps)
    return o


class DenseLayerC(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in
                ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "gate", "up", "down")]


def dense_decode_layer(layer: dict, x, kc: np.ndarray, vc: np.ndarray, pos: int, heads: int, kv_heads: int, hd: int,
                       ff: int, eps: float, rope_base: float, attn_scale: float, mode: int = MUL_ADD,
                       pool: Pool | None = None) -> np.ndarray:
    """One Llama-shaped layer for one new token (ref/dense.zig:134-146); kc/vc (uint16 f16 bits) get row `pos`."""
    x = _f32(x).copy()
    e = x.size
    keep = {k: _f32(layer[k]) for k in ("attn_norm", "ffn_norm")}
    s = DenseLayerC(_p(keep["attn_norm"]).value, layer["wq"].h, layer["wk"].h, layer["wv"].h, layer["wo"].h,
                    _p(keep["ffn_norm"]).value, layer["gate"].h, layer["up"].h, layer["down"].h)
    assert kc.dtype == np.uint16 and vc.dtype == np.uint16 and kc.flags.c_contiguous and vc.flags.c_contiguous
    lib().ref_dense_decode_layer((pool or default_pool()).h, C.byref(s), _p(x), _p(kc), _p(vc), pos, e, heads, kv_heads,
                                 hd, ff, eps, rope_base, attn_scale, mode)
    return x


def dense_head(x, out_norm, head: Matrix, eps: float, mode: int = MUL_ADD, pool: Pool | None = None) -> np.ndarray:
    x, out_norm = _f32(x), _f32(out_norm)
    logits = np.empty(head.n, dtype=np.float32)
    lib().ref_dense_head((pool or default_pool()).h, _p(logits), _p(x), _p(out_norm), head.h, x.size, eps, mode)
    return logits


def build_info() -> str:
    return lib().ref_build_info().decode()
