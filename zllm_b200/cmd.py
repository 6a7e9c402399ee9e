"""The command stream a zllm core hands to a GPU host, restated from
src/gpu/cmd.zig:21-203: little-endian u32 words, header `opcode | words << 8`,
ids dense per kind and assigned by the recorder, host addresses as two words.
Used to drive zcu_execute the way the Zig plan would.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

CREATE_BUFFER, WRITE_BUFFER, CREATE_KERNEL, CREATE_BIND_GROUP, DISPATCH = 1, 2, 3, 5, 6
COPY_BUFFER, READ_BUFFER, SUBMIT, DESTROY, CLEAR_BUFFER, WRITE_FILE = 7, 8, 9, 10, 11, 12

# cmd.Usage bits (WebGPU GPUBufferUsage)
COPY_SRC, COPY_DST, UNIFORM, STORAGE = 1 << 2, 1 << 3, 1 << 6, 1 << 7
KIND_BUFFER, KIND_PIPELINE, KIND_BIND_GROUP = 0, 1, 2


def _split(v: int):
    return [v & 0xFFFFFFFF, (v >> 32) & 0xFFFFFFFF]


class Recorder:
    """cmd.Recorder: appends commands; `batch()` is what a host executes."""

    def __init__(self):
        self.words: list[int] = []
        self.next = [0, 0, 0]
        self._keep = []  # host arrays the recorded addresses point into

    def batch(self) -> np.ndarray:
        return np.array(self.words, dtype=np.uint32)

    def clear(self):
        self.words = []
        self._keep = []

    def _put(self, op: int, args):
        self.words.append(op | ((len(args) + 1) << 8))
        self.words.extend(int(a) & 0xFFFFFFFF for a in args)

    def _alloc(self, kind: int) -> int:
        i = self.next[kind]
        self.next[kind] += 1
        return i

    def create_buffer(self, size: int, usage: int = STORAGE | COPY_SRC | COPY_DST) -> int:
        i = self._alloc(KIND_BUFFER)
        self._put(CREATE_BUFFER, [i] + _split(size) + [usage])
        return i

    def write_buffer(self, buffer: int, offset: int, data: np.ndarray):
        a = np.ascontiguousarray(data)
        self._keep.append(a)
        self._put(WRITE_BUFFER, [buffer] + _split(offset) + _split(a.ctypes.data) + _split(a.nbytes))

    def write_file(self, buffer: int, offset: int, file_offset: int, size: int):
        self._put(WRITE_FILE, [buffer] + _split(offset) + _split(file_offset) + _split(size))

    def create_kernel(self, kernel: int, variant: int, writes: int, artifact: bytes) -> int:
        i = self._alloc(KIND_PIPELINE)
        buf = C.create_string_buffer(artifact, max(1, len(artifact)))
        self._keep.append(buf)
        self._put(CREATE_KERNEL, [i, kernel, variant, writes] + _split(C.addressof(buf)) + [len(artifact)])
        return i

    def create_bind_group(self, pipeline: int, entries) -> int:
        """entries: [(binding, buffer, offset, size)]."""
        i = self._alloc(KIND_BIND_GROUP)
        args = [i, pipeline, 0, len(entries)]
        for binding, buffer, offset, size in entries:
            args += [binding, buffer] + _split(offset) + _split(size)
        self._put(CREATE_BIND_GROUP, args)
        return i

    def dispatch(self, pipeline: int, groups, bind_groups):
        self._put(DISPATCH, [pipeline, groups[0], groups[1], groups[2], len(bind_groups)] + list(bind_groups))

    def copy_buffer(self, src: int, src_offset: int, dst: int, dst_offset: int, size: int):
        self._put(COPY_BUFFER, [src] + _split(src_offset) + [dst] + _split(dst_offset) + _split(size))

    def clear_buffer(self, buffer: int, offset: int, size: int):
        self._put(CLEAR_BUFFER, [buffer] + _split(offset) + _split(size))

    def read_buffer(self, token: int, buffer: int, offset: int, dst: np.ndarray):
        assert dst.flags.c_contiguous
        self._keep.append(dst)
        self._put(READ_BUFFER, [token, buffer] + _split(offset) + _split(dst.nbytes) + _split(dst.ctypes.data))

    def submit(self, token: int):
        self._put(SUBMIT, [token])

    def destroy(self, kind: int, i: int):
        self._put(DESTROY, [kind, i])


def iterate(words):
    """cmd.Iterator: yields (op, args) and raises ValueError('Truncated'|'BadLength')."""
    pos, n = 0, len(words)
    while pos < n:
        word = int(words[pos])
        length = word >> 8
        if length == 0:
            raise ValueError("BadLength")
        if length > n - pos:
            raise ValueError("Truncated")
        yield word & 0xFF, [int(w) for w in words[pos + 1:pos + length]]
        pos += length
