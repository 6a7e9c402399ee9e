"""ctypes binding of include/zllm_cuda.h (libzllm_cuda.so).

There is no CPU path: loading fails loudly when the library has not been
built, and creating a context fails when there is no sm_100 device (except
for an explicit dry run, which executes no kernel).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libzllm_cuda.so"

ABI_VERSION = 1

OK = 0
E_GPU, E_DEVICE_LOST, E_BAD_COMMAND, E_BAD_ID, E_NO_TIMESTAMPS = -1, -2, -3, -4, -5
E_UNSUPPORTED_KERNEL, E_UNSUPPORTED_PREFILL, E_TRUNCATED, E_BAD_LENGTH = -6, -7, -8, -9
E_OUT_OF_MEMORY, E_TIMEOUT, E_INVALID = -10, -11, -12

ERROR_NAMES = {
    E_GPU: "GpuError", E_DEVICE_LOST: "DeviceLost", E_BAD_COMMAND: "BadCommand", E_BAD_ID: "BadId",
    E_NO_TIMESTAMPS: "NoTimestamps", E_UNSUPPORTED_KERNEL: "UnsupportedKernel",
    E_UNSUPPORTED_PREFILL: "UnsupportedPrefill", E_TRUNCATED: "Truncated", E_BAD_LENGTH: "BadLength",
    E_OUT_OF_MEMORY: "OutOfMemory", E_TIMEOUT: "Timeout", E_INVALID: "Invalid",
}

# Every symbol include/zllm_cuda.h declares.
EXPORTS = [
    "zcu_create", "zcu_destroy", "zcu_get_caps", "zcu_last_error", "zcu_force_loss", "zcu_memory_budget",
    "zcu_backend_source", "zcu_artifact", "zcu_supports_prefill", "zcu_execute", "zcu_set_file",
    "zcu_start_profile", "zcu_stop_profile", "zcu_read_timings", "zcu_alloc", "zcu_free", "zcu_upload",
    "zcu_download", "zcu_memset", "zcu_launch", "zcu_sync", "zcu_launch_count", "zcu_capture_begin",
    "zcu_capture_end", "zcu_graph_launch", "zcu_graph_destroy", "zcu_rope_table",
    "zcu_attention_decode_static", "zcu_peer_wait_limit", "zcu_ipc_export", "zcu_ipc_open", "zcu_peer_config",
]


class Options(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("device_index", C.c_uint32), ("dry_run", C.c_uint32),
                ("reserved", C.c_uint32), ("stream", C.c_void_p)]


class Caps(C.Structure):
    _fields_ = [("abi_version", C.c_uint32), ("sm_major", C.c_uint32), ("sm_minor", C.c_uint32),
                ("sm_count", C.c_uint32), ("max_shared_per_block", C.c_uint32), ("l2_bytes", C.c_uint32),
                ("total_bytes", C.c_uint64), ("free_bytes", C.c_uint64), ("max_binding_lo", C.c_uint32),
                ("max_binding_hi", C.c_uint32), ("offset_align", C.c_uint32), ("dry_run", C.c_uint32),
                ("device_name", C.c_char * 128)]


class Completion(C.Structure):
    _fields_ = [("token", C.c_uint32), ("status", C.c_uint32)]


class Binding(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("size", C.c_uint64)]


class Timing(C.Structure):
    _fields_ = [("kernel", C.c_uint32), ("variant", C.c_uint32), ("grid", C.c_uint32 * 3), ("count", C.c_uint32),
                ("total_us", C.c_double)]


class ZcuError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code
        self.name = ERROR_NAMES.get(code, str(code))
        self.message = message


_lib = None


def lib() -> C.CDLL:
    """Loads libzllm_cuda.so; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m zllm_b200.build` "
                           "(there is no CPU implementation to fall back to)")
    L = C.CDLL(str(LIB_PATH))
    vp, u32, u64, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_size_t
    sig = {
        "zcu_create": (C.c_int32, [C.POINTER(Options), C.POINTER(vp)]),
        "zcu_destroy": (C.c_int32, [vp, u32]),
        "zcu_get_caps": (C.c_int32, [vp, C.POINTER(Caps)]),
        "zcu_last_error": (sz, [vp, C.c_char_p, sz]),
        "zcu_force_loss": (C.c_int32, [vp]),
        "zcu_memory_budget": (C.c_int32, [vp, C.POINTER(u64)]),
        "zcu_backend_source": (C.c_char_p, []),
        "zcu_artifact": (sz, [u32, u32, C.c_char_p, sz]),
        "zcu_supports_prefill": (C.c_int32, [vp, u32]),
        "zcu_execute": (C.c_int32, [vp, vp, sz, C.POINTER(Completion), sz, C.POINTER(sz), u32]),
        "zcu_set_file": (C.c_int32, [vp, vp, u64, C.c_char_p]),
        "zcu_start_profile": (C.c_int32, [vp]),
        "zcu_stop_profile": (C.c_int32, [vp]),
        "zcu_read_timings": (C.c_int32, [vp, C.POINTER(Timing), sz, C.POINTER(sz)]),
        "zcu_alloc": (C.c_int32, [vp, u64, C.POINTER(vp)]),
        "zcu_free": (C.c_int32, [vp, vp]),
        "zcu_upload": (C.c_int32, [vp, vp, vp, u64]),
        "zcu_download": (C.c_int32, [vp, vp, vp, u64]),
        "zcu_memset": (C.c_int32, [vp, vp, C.c_int, u64]),
        "zcu_launch": (C.c_int32, [vp, u32, u32, vp, u32, C.POINTER(Binding), u32, C.POINTER(u32)]),
        "zcu_sync": (C.c_int32, [vp, u32]),
        "zcu_launch_count": (u64, [vp]),
        "zcu_peer_wait_limit": (C.c_int32, [vp, u32]),
        "zcu_capture_begin": (C.c_int32, [vp]),
        "zcu_capture_end": (C.c_int32, [vp, C.POINTER(u32)]),
        "zcu_graph_launch": (C.c_int32, [vp, u32]),
        "zcu_graph_destroy": (C.c_int32, [vp, u32]),
        "zcu_rope_table": (C.c_int32, [vp, u32, u32, C.c_float, vp]),
        "zcu_attention_decode_static": (C.c_int32, [vp, vp, u32, C.POINTER(Binding), u32, u32, u32]),
        "zcu_ipc_export": (C.c_int32, [vp, vp, vp]),
        "zcu_ipc_open": (C.c_int32, [vp, vp, C.POINTER(vp)]),
        "zcu_peer_config": (C.c_int32, [vp, u32, u32, C.POINTER(u64), u64, u64, u32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def artifact(kernel: int, variant: int = 0) -> bytes:
    """kernels.artifact(.cuda, k, variant): empty for an identity this backend lacks."""
    buf = C.create_string_buffer(64)
    n = lib().zcu_artifact(kernel, variant, buf, 64)
    return buf.value if n else b""


def rope_table(positions: int, n_rot: int, base: float, factors=None) -> np.ndarray:
    """kernels.ropeTableScaled: the (cos, sin) table rope_append reads, built on the host in f32."""
    out = np.empty(positions * (n_rot // 2) * 2, dtype=np.float32)
    f = None if factors is None else np.ascontiguousarray(factors, dtype=np.float32)
    r = lib().zcu_rope_table(out.ctypes.data, positions, n_rot, base, None if f is None else f.ctypes.data)
    if r != OK:
        raise ZcuError(r, "zcu_rope_table: bad arguments")
    return out


def backend_source() -> str:
    return lib().zcu_backend_source().decode()


class DevBuf:
    """A device allocation made through zcu_alloc."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx, self.nbytes = ctx, int(nbytes)
        p = C.c_void_p()
        ctx._check(lib().zcu_alloc(ctx.h, self.nbytes, C.byref(p)))
        self.ptr = p.value

    def upload(self, arr: np.ndarray, offset: int = 0) -> "DevBuf":
        a = np.ascontiguousarray(arr)
        assert offset + a.nbytes <= max(self.nbytes, 256), (offset, a.nbytes, self.nbytes)
        self.ctx._check(lib().zcu_upload(self.ctx.h, self.ptr + offset, a.ctypes.data, a.nbytes))
        self.ctx.sync()  # the source array may go away after this returns
        return self

    def download(self, dtype, count: int | None = None, offset: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        n = (self.nbytes - offset) // dt.itemsize if count is None else count
        out = np.empty(n, dtype=dt)
        self.ctx._check(lib().zcu_download(self.ctx.h, out.ctypes.data, self.ptr + offset, out.nbytes))
        return out

    def zero(self) -> "DevBuf":
        self.ctx._check(lib().zcu_memset(self.ctx.h, self.ptr, 0, self.nbytes))
        return self

    def at(self, offset: int = 0, size: int | None = None) -> tuple[int, int]:
        return (self.ptr + offset, self.nbytes - offset if size is None else size)

    def free(self):
        if self.ptr:
            lib().zcu_free(self.ctx.h, self.ptr)
            self.ptr = None


class SubBuf(DevBuf):
    """A range of a larger device allocation (an arena), with DevBuf's interface."""

    def __init__(self, ctx: "Context", ptr: int, nbytes: int):  # no allocation of its own
        self.ctx, self.ptr, self.nbytes = ctx, int(ptr), int(nbytes)

    def free(self):
        self.ptr = None


class PeerArena:
    """One rank's arena for the tensor-parallel exchange over peer memory (include/zllm_cuda.h): the vectors
    every rank reads whole, then their tagged exchange slots. `exchange(handle_bytes) -> [handle_bytes per rank]` is the
    caller's all-gather of the 64-byte IPC handles (torch.distributed.all_gather_object, or anything else);
    with world == 1 nothing is exchanged."""

    def __init__(self, ctx: "Context", rank: int, world: int, data_bytes: int, slots: int, exchange=None):
        self.ctx, self.rank, self.world, self.slots = ctx, rank, world, slots
        self.data_bytes = (int(data_bytes) + 255) & ~255
        self.nbytes = 3 * self.data_bytes  # the vectors, then 8 bytes {value, tag} per float of them
        self.buf = ctx.alloc(self.nbytes).zero()
        ctx.sync()
        bases = [0] * world
        bases[rank] = self.buf.ptr
        if world > 1:
            handle = C.create_string_buffer(64)
            ctx._check(lib().zcu_ipc_export(ctx.h, self.buf.ptr, handle))
            handles = exchange(handle.raw)
            for r in range(world):
                if r != rank:
                    p = C.c_void_p()
                    ctx._check(lib().zcu_ipc_open(ctx.h, C.create_string_buffer(handles[r], 64), C.byref(p)))
                    bases[r] = p.value
        arr = (C.c_uint64 * world)(*bases)
        ctx._check(lib().zcu_peer_config(ctx.h, rank, world, arr, self.nbytes, self.data_bytes, slots))
        self.bases, self.used = bases, 0

    def alloc(self, nbytes: int) -> SubBuf:
        size = (int(nbytes) + 255) & ~255
        assert self.used + size <= self.data_bytes, "the arena is full"
        b = SubBuf(self.ctx, self.buf.ptr + self.used, nbytes)
        self.used += size
        return b


class Context:
    """One zcu_context: a device (or a dry run) and its stream."""

    def __init__(self, device: int = 0, dry_run: bool = False, stream: int | None = None):
        opts = Options(ABI_VERSION, device, int(dry_run), 0, stream)
        h = C.c_void_p()
        r = lib().zcu_create(C.byref(opts), C.byref(h))
        if r != OK:
            raise ZcuError(r, "zcu_create failed: no sm_100 CUDA device (this backend has no CPU path)")
        self.h = h
        self.dry_run = dry_run
        self._bufs: list[DevBuf] = []

    # -- errors
    def last_error(self) -> str:
        buf = C.create_string_buffer(1024)
        lib().zcu_last_error(self.h, buf, 1024)
        return buf.value.decode(errors="replace")

    def _check(self, r: int):
        if r != OK:
            raise ZcuError(r, self.last_error())

    # -- info
    def caps(self) -> Caps:
        c = Caps()
        self._check(lib().zcu_get_caps(self.h, C.byref(c)))
        return c

    def memory_budget(self) -> int:
        v = C.c_uint64()
        self._check(lib().zcu_memory_budget(self.h, C.byref(v)))
        return v.value

    def supports_prefill(self, rung_variant: int) -> bool:
        """Device.supportsPrefill (src/gpu/host.zig:120-128) for a rung's reserved variant id."""
        return bool(lib().zcu_supports_prefill(self.h, rung_variant))

    def force_loss(self):
        self._check(lib().zcu_force_loss(self.h))

    # -- memory
    def alloc(self, nbytes: int) -> DevBuf:
        b = DevBuf(self, nbytes)
        self._bufs.append(b)
        return b

    def put(self, arr: np.ndarray) -> DevBuf:
        a = np.ascontiguousarray(arr)
        return self.alloc(max(a.nbytes, 4)).upload(a)

    def zeros(self, nbytes: int) -> DevBuf:
        return self.alloc(nbytes).zero()

    # -- work
    def launch(self, kernel: int, params, bindings, grid, variant: int = 0):
        """bindings: sequence of DevBuf | (ptr, size) | None, binding 1 first."""
        pb = bytes(params)
        arr = (Binding * max(1, len(bindings)))()
        for i, b in enumerate(bindings):
            if b is None:
                arr[i] = Binding(None, 0)
            elif hasattr(b, "ptr") and hasattr(b, "nbytes"):  # a DevBuf, or any buffer object of the caller
                arr[i] = Binding(b.ptr, b.nbytes)
            else:
                arr[i] = Binding(b[0], b[1])
        g = (C.c_uint32 * 3)(*grid)
        self._check(lib().zcu_launch(self.h, kernel, variant, pb, len(pb), arr, len(bindings), g))

    def attention_decode_static(self, params, bindings, max_keys: int, rows: int):
        """attn_split + attn_combine with the partials in the library's fixed 4 MiB array: for callers that
        cannot allocate device memory. bindings: qg, kc, vc, out, step [, positions]."""
        pb = bytes(params)
        arr = (Binding * len(bindings))()
        for i, b in enumerate(bindings):
            arr[i] = Binding(b.ptr, b.nbytes) if hasattr(b, "ptr") else Binding(b[0], b[1])
        self._check(lib().zcu_attention_decode_static(self.h, pb, len(pb), arr, len(bindings), max_keys, rows))

    def sync(self, timeout_ms: int = 60000):
        self._check(lib().zcu_sync(self.h, timeout_ms))

    def peer_wait_limit(self, milliseconds: int):
        self._check(lib().zcu_peer_wait_limit(self.h, milliseconds))

    def launch_count(self) -> int:
        return lib().zcu_launch_count(self.h)

    def execute(self, words: np.ndarray, timeout_ms: int = 60000, cap: int = 4096):
        """Runs one command-stream batch; returns [(token, status)]. Raises ZcuError."""
        w = np.ascontiguousarray(words, dtype=np.uint32)
        out = (Completion * cap)()
        n = C.c_size_t()
        r = lib().zcu_execute(self.h, w.ctypes.data, w.size, out, cap, C.byref(n), timeout_ms)
        done = [(out[i].token, out[i].status) for i in range(min(n.value, cap))]
        if r != OK:
            e = ZcuError(r, self.last_error())
            e.completions = done
            raise e
        return done

    def set_file(self, data: np.ndarray, path: str = ""):
        self._file = np.ascontiguousarray(data).view(np.uint8)
        self._check(lib().zcu_set_file(self.h, self._file.ctypes.data, self._file.nbytes, path.encode()))

    def start_profile(self):
        self._check(lib().zcu_start_profile(self.h))

    def stop_profile(self):
        self._check(lib().zcu_stop_profile(self.h))

    def timings(self):
        n = C.c_size_t()
        self._check(lib().zcu_read_timings(self.h, None, 0, C.byref(n)))
        out = (Timing * max(1, n.value))()
        self._check(lib().zcu_read_timings(self.h, out, n.value, C.byref(n)))
        return [(t.kernel, t.variant, tuple(t.grid), t.count, t.total_us) for t in out[: n.value]]

    # -- graphs
    def capture_begin(self):
        self._check(lib().zcu_capture_begin(self.h))

    def capture_end(self) -> int:
        g = C.c_uint32()
        self._check(lib().zcu_capture_end(self.h, C.byref(g)))
        return g.value

    def graph_launch(self, graph: int):
        self._check(lib().zcu_graph_launch(self.h, graph))

    def graph_destroy(self, graph: int):
        self._check(lib().zcu_graph_destroy(self.h, graph))

    def close(self):
        if self.h:
            for b in self._bufs:
                b.free()
            self._bufs.clear()
            lib().zcu_destroy(self.h, 60000)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
