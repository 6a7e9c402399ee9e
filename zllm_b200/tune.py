"""Load-time tuning of the quantised decode multiplies: the counterpart of the reference's tune.Sweep
(src/tune/tune.zig:1-27, 77-106). For each shape (type, n, k) every candidate variant of this backend
(kernels.MATVEC_CANDIDATES: tiles in flight per warp, CTA shape and CTA count of the tensor-core family, and the
scalar family) runs on the shape's real weights: it is first checked against the default variant (relative L2 error above `TOLERANCE`
drops it: candidates differ only in the order of each row's sums), then timed - `WARMUP` batches, then the median
of `TIMED` batches, each batch repeating the dispatch so that it lasts about a millisecond and replayed as a CUDA
graph, the way a plan replays its step. The fastest per shape
goes into the table a plan passes as `variants`.

The inputs are the reference's: x[i] = sin(0.7 i), of RMS about 1 like normed activations."""
from __future__ import annotations

import time

import numpy as np

from . import kernels as K

TIMED, WARMUP, TOLERANCE = 7, 3, 1e-5  # src/tune/tune.zig:24-30


def _rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    den = float(np.sqrt((want.astype(np.float64) ** 2).sum()))
    return float(np.sqrt(((got.astype(np.float64) - want.astype(np.float64)) ** 2).sum())) / (den if den > 0 else 1.0)


class Sweep:
    """sweep = Sweep(ctx, tokens=1); sweep.add("q4_k", weights_buffer, n, k); table = sweep.run()"""

    def __init__(self, ctx, tokens: int = 1, candidates=None):
        assert 1 <= tokens <= 4  # kernels.decode_max_rows
        self.ctx, self.tokens = ctx, tokens
        self.candidates = list(candidates if candidates is not None else [0] + K.MATVEC_CANDIDATES)
        assert self.candidates[0] == 0, "the default first: it is the reference the others must match"
        self.shapes, self.dropped, self.report = [], 0, []
        self.L = K.Launcher(ctx)
        self._graph = None   # ((shape, variant), graph) of the batch captured last

    def add(self, ttype: str, weights, n: int, k: int, **flags):
        """`weights`: the shape's matrix, or a list of matrices of this shape (every layer's): a batch then rotates
        through them, so that a shape smaller than L2 is still timed from HBM, where a decode step finds it.
        `flags`: what the plan passes with this shape (flags, eps, half, norm_w), so that the variant is timed as used."""
        if ttype not in ("q4_k", "q8_0") or any(s[0] == ttype and s[2] == n and s[3] == k for s in self.shapes):
            return
        ws = list(weights) if isinstance(weights, list) else [weights]
        if "flags" in flags:
            flags["flags"] &= ~K.ACCUMULATE   # every run must give the same output: nothing accumulates in the sweep
        row_bytes = K.row_bytes(ttype, k)
        rows = n + (flags.get("half", 0) if flags.get("flags", 0) & K.SILU_PAIR else 0)
        reps = int(np.clip((256 << 20) // max(rows * row_bytes, 1), 2, 64))
        self.shapes.append((ttype, ws, n, k, reps, flags))

    def _batch(self, shape, variant, x, out) -> float:
        """Seconds per dispatch of one batch. The batch is replayed as a CUDA graph (captured on its first use), as a
        plan replays its step: the dispatches then follow each other on the device the way they do in a step, and the
        host's launch cost stays out of the figure."""
        ttype, ws, n, k, reps, flags = shape
        key = (id(shape), variant)
        if self._graph is None or self._graph[0] != key:
            if self._graph is not None:
                self.ctx.graph_destroy(self._graph[1])
                self._graph = None
            self.ctx.capture_begin()
            try:
                for i in range(reps):
                    self.L.matvec(ttype, x, ws[i % len(ws)], out, n, k, m=self.tokens, variant=variant, **flags)
            finally:
                g = self.ctx.capture_end()
            self._graph = (key, g)
        self.ctx.sync()
        t0 = time.perf_counter()
        self.ctx.graph_launch(self._graph[1])
        self.ctx.sync()
        return (time.perf_counter() - t0) / reps

    def run(self) -> dict:
        """{(type, n, k): variant word} with the fastest agreeing candidate of every shape."""
        table = {}
        if not self.shapes:
            return table
        k_max = max(s[3] for s in self.shapes)
        n_max = max(s[2] for s in self.shapes)
        xs = np.sin(np.arange(self.tokens * k_max, dtype=np.float32) * np.float32(0.7)).astype(np.float32)
        out = self.ctx.zeros(self.tokens * n_max * 4)
        for shape in self.shapes:
            ttype, _, n, k, reps, _ = shape
            x = self.ctx.put(xs[: self.tokens * k])
            reference, best = None, None
            for variant in self.candidates:
                if not K.matvec_variant_exists(ttype, k, variant):
                    continue
                self._batch(shape, variant, x, out)  # the correctness run is the first warm-up batch
                got = out.download(np.float32, self.tokens * n)
                if reference is None:
                    reference = got.copy()
                elif _rel_l2(got, reference) > TOLERANCE or not np.isfinite(got).all():
                    self.dropped += 1
                    self.report.append((ttype, n, k, variant, None))
                    continue
                for _ in range(WARMUP - 1):
                    self._batch(shape, variant, x, out)
                ns = float(np.median([self._batch(shape, variant, x, out) for _ in range(TIMED)])) * 1e9
                self.report.append((ttype, n, k, variant, ns))
                if best is None or ns < best[1]:
                    best = (variant, ns)
            table[(ttype, n, k)] = best[0]
        if self._graph is not None:
            self.ctx.graph_destroy(self._graph[1])
            self._graph = None
        return table
