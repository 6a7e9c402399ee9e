"""PyTorch as plumbing: torch tensors as plan buffers, and the NCCL all-gather of column slices.
Only the multi-GPU paths and the benchmark import this module."""
from __future__ import annotations

import numpy as np


class TorchBuf:
    """A zeroed torch uint8 tensor as a device buffer: .ptr/.nbytes for bindings, upload() for inputs."""

    def __init__(self, torch, dev, nbytes: int):
        self.t = torch.zeros(max(int(nbytes), 256), dtype=torch.uint8, device=dev)
        self.ptr, self.nbytes, self.torch = self.t.data_ptr(), int(nbytes), torch

    def upload(self, arr: np.ndarray, offset: int = 0):
        src = self.torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1))
        self.t[offset:offset + src.numel()].copy_(src, non_blocking=False)
        return self

    def download(self, dtype, count=None, offset: int = 0) -> np.ndarray:
        raw = self.t[offset:self.nbytes].cpu().numpy().view(dtype)
        return raw if count is None else raw[:count]

    def at(self, offset: int = 0, size=None):
        return (self.ptr + offset, self.nbytes - offset if size is None else size)

    def f32(self):
        return self.t[: self.nbytes].view(self.torch.float32)


def nccl_gather(dist, rank: int, world: int):
    """gather(buf, batch, width): every rank's column slice [rank*width/world, ...) of each row of a
    [batch, width] f32 buffer becomes visible on all ranks (in-place all-gather, one per row)."""

    def gather(buf, batch, width):
        t = buf.f32().view(batch, width)
        per = width // world
        for b in range(batch):
            dist.all_gather_into_tensor(t[b], t[b, rank * per:(rank + 1) * per])

    return gather
