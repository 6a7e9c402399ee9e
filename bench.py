"""Benchmark of the CUDA backend's hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line on stdout (rank 0). Workloads:
  matvec_q4_k  the Q4_K decode multiply at the Llama-3-8B FFN-up shape (14336 x 4096, batch 1):
               a step is one pass over R distinct weight matrices (R * 33 MB > L2), metric = HBM GB/s.
  decode       one decode step of the Llama-3-8B-shaped Q4_K model at context 8192, metric = tokens/s.
`--impl reference` times the CPU oracle (the restatement of the reference's own CPU path) on the host
cores instead, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

PEAKS_FILE = ROOT / "MEASURED_PEAKS.json"
FALLBACK_HBM_GBS = 6650.0


def measured_hbm_peak():
    try:
        return float(json.loads(PEAKS_FILE.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s: the burst figure (a kernel timed alone over a short region)."""
    try:
        return float(json.loads(PEAKS_FILE.read_text())["bf16_tflops"]), "measured (burst)"
    except Exception:
        return 1590.0, "fallback"


# ------------------------------------------------------------------ clocks

class ClockSampler:
    """Samples the SM clock and the throttle reasons while the timed region runs: NVML read calls from a thread every
    5 ms (a 20-step decode run lasts 40 ms: nvidia-smi's own loop would see it once at most); nvidia-smi as the
    fallback where the NVML binding is missing. Reads only: no setting of the device is touched."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    # nvmlClocksEventReasons bits
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, device: int):
        self.device = device
        self.proc = None
        self.path = None
        self.thread = None
        self.sm, self.mx, self.reasons = [], [], set()

    def _nvml_loop(self, nv, handle):
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                self.mx.append(float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM)))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = int(get(handle))
                for name, bit in self.REASON_BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001 - a failed read is a missing sample
                pass
            self._stop.wait(0.005)

    def start(self):
        try:
            import threading

            import pynvml as nv

            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.device]) if visible and visible.replace(",", "").isdigit() else self.device
            handle = nv.nvmlDeviceGetHandleByIndex(index)
            self._stop = threading.Event()
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:  # noqa: BLE001 - no NVML binding: nvidia-smi below
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.device)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            if self.sm:
                out.update(sm_mhz=float(np.median(self.sm)), sm_max_mhz=float(max(self.mx)), samples=len(self.sm), source="nvml")
            out["reasons"] = sorted(self.reasons)
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(mx))
            out["samples"] = len(sm)
            out["source"] = "nvidia-smi"
        out["reasons"] = sorted(reasons)
        return out


# ------------------------------------------------------------------ distributed plumbing

class Dist:
    def __init__(self, gpus: int):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.on = self.world > 1
        if self.on:
            import torch
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            torch.cuda.set_device(self.local)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist
        if gpus != self.world and self.rank == 0 and self.on:
            print(f"bench: --gpus {gpus} but WORLD_SIZE {self.world}; using {self.world}", file=sys.stderr)

    def barrier(self):
        if self.on:
            self.dist.barrier()

    def max(self, value: float) -> float:
        if not self.on:
            return value
        import torch

        t = torch.tensor([value], dtype=torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def max_each(self, values):
        """Element-wise maximum over ranks of a short list of floats (every rank passes the same count)."""
        if not self.on:
            return list(values)
        import torch

        t = torch.tensor(list(values), dtype=torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.on:
            self.dist.destroy_process_group()


# ------------------------------------------------------------------ workload: Q4_K matvec

class MatvecQ4K:
    """configs[1]: x f32[batch, 4096] ~ N(0,1); W Q4_K [14336 x 4096]; out f32[batch, 14336].
    With N ranks the rows of every matrix are sharded (rank r owns rows [r*n/N, (r+1)*n/N)) and the
    output slices are all-gathered over NCCL."""

    n, k = 14336, 4096
    name = "matvec_q4_k"

    def __init__(self, dist: Dist, batch: int = 1, variant: int = 0, tune: bool = True, **_):
        import torch

        from zllm_b200 import abi, synth
        from zllm_b200 import kernels as K

        self.torch, self.K, self.dist, self.batch, self.variant = torch, K, dist, batch, variant
        # more than four tokens: one pass over the weights by the batched tcgen05 family (unless a variant was asked for;
        # --variant 0x20000 = a pass per 2-4 tokens by the mma.sync family)
        if variant == 0 and 4 < batch <= K.MATVEC_BATCHED_MAX_TOKENS:
            self.variant = K.MATVEC_BATCHED
        self.dev = torch.device("cuda", dist.local)
        torch.cuda.set_device(self.dev)
        self.stream = torch.cuda.Stream(self.dev)
        self.ctx = abi.Context(dist.local, stream=self.stream.cuda_stream)
        self.launcher = K.Launcher(self.ctx)
        self.copies = 8 * dist.world                     # per-rank footprint stays above the 126 MB L2
        self.rows = self.n // dist.world
        rb = K.row_bytes("q4_k", self.k)
        rng = synth.rng_for("cfg2", f"w-rank{dist.rank}")
        one = synth.q4_k_weights(rng, self.rows, self.k)
        self.host_w0 = one
        self.w = torch.empty((self.copies, self.rows * rb), dtype=torch.uint8, device=self.dev)
        base = torch.from_numpy(one.reshape(-1)).to(self.dev)
        for c in range(self.copies):
            # distinct bytes per copy (a rotation of the rows) so no two copies can share cache lines
            self.w[c] = torch.roll(base.view(self.rows, rb), shifts=c, dims=0).reshape(-1)
        self.host_x = synth.normal_f32(synth.rng_for("cfg2", f"x{batch}"), batch, self.k)
        self.pinned_x = torch.from_numpy(self.host_x).pin_memory()
        self.x = self.pinned_x.to(self.dev)
        self.out = torch.zeros((self.copies, batch, self.n), dtype=torch.float32, device=self.dev)
        self.local_out = torch.zeros((self.copies, batch, self.rows), dtype=torch.float32, device=self.dev)
        self.pinned_out = torch.empty((batch, self.n), dtype=torch.float32).pin_memory()
        self.graph = None
        torch.cuda.synchronize()
        # the load-time sweep over the multiply's variants on this shape (src/tune/tune.zig), unless one was asked for
        self.tuned = None
        if variant == 0 and batch <= 4 and tune:
            from zllm_b200 import tune as T

            sweep = T.Sweep(self.ctx, tokens=batch)
            sweep.add("q4_k", [(self.w[c].data_ptr(), self.w[c].numel()) for c in range(self.copies)], self.rows, self.k)
            self.variant = self.tuned = sweep.run()[("q4_k", self.rows, self.k)]
            torch.cuda.synchronize()

    # algorithmic bytes of one launch on one rank (weights + x + out)
    def bytes_per_launch(self) -> int:
        return self.rows * (self.k // 256) * 144 + 4 * self.batch * self.k + 4 * self.batch * self.rows

    def launches_per_step(self) -> int:
        return self.copies

    def units_per_step(self) -> float:
        """Whole-job algorithmic bytes of a step."""
        return float(self.bytes_per_launch() * self.copies * self.dist.world)

    def _launch_all(self):
        K = self.K
        for c in range(self.copies):
            if self.dist.on:
                dst = (self.local_out[c].data_ptr(), self.local_out[c].numel() * 4)
                self.launcher.matvec("q4_k", (self.x.data_ptr(), self.x.numel() * 4),
                                     (self.w[c].data_ptr(), self.w[c].numel()), dst, self.rows, self.k, m=self.batch, variant=self.variant)
            else:
                self.launcher.matvec("q4_k", (self.x.data_ptr(), self.x.numel() * 4),
                                     (self.w[c].data_ptr(), self.w[c].numel()),
                                     (self.out[c].data_ptr(), self.out[c].numel() * 4), self.n, self.k, m=self.batch,
                                     variant=self.variant)

    def step(self):
        """One pass over every weight copy, inputs resident in HBM."""
        if not self.dist.on:
            if self.graph is None:
                self.ctx.capture_begin()
                self._launch_all()
                self.graph = self.ctx.capture_end()
            self.ctx.graph_launch(self.graph)
            return
        torch = self.torch
        with torch.cuda.stream(self.stream):
            self._launch_all()
            for c in range(self.copies):
                # gather the row slices: out[c][b][r*rows:(r+1)*rows] <- rank r
                gathered = torch.empty((self.dist.world, self.batch, self.rows), dtype=torch.float32, device=self.dev)
                self.dist.dist.all_gather_into_tensor(gathered, self.local_out[c])
                self.out[c] = gathered.permute(1, 0, 2).reshape(self.batch, self.n)

    def e2e_step(self):
        """The same pass through the user-facing path: x comes from pinned host memory and the last
        matrix's output goes back to the host, inside the timed region."""
        torch = self.torch
        with torch.cuda.stream(self.stream):
            self.x.copy_(self.pinned_x, non_blocking=True)
        self.step()
        with torch.cuda.stream(self.stream):
            self.pinned_out.copy_(self.out[self.copies - 1], non_blocking=True)
        self.stream.synchronize()

    def e2e_bytes(self):
        return self.host_x.nbytes, self.pinned_out.numel() * 4

    def roofline(self, ms_per_step: float):
        peak, kind = measured_hbm_peak()
        us = ms_per_step * 1e3 / self.launches_per_step()
        achieved = self.bytes_per_launch() / us / 1e3
        kernel = "qgemm_q4k_kernel (tcgen05; with its column and reduction kernels)" if self.variant == self.K.MATVEC_BATCHED else "matvec_imma<Q4_K>"
        return {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {kind}", "frac_of_8000_nominal": achieved / 8000.0,
                "traffic": None, "bytes_per_launch": self.bytes_per_launch(), "us_per_launch": us}

    def metric(self):
        return "q4_k_matvec_hbm_gbs", "GB/s"

    def value(self, seconds_per_step: float) -> float:
        return self.units_per_step() / seconds_per_step / 1e9

    def config(self):
        return {"workload": f"Q4_K matvec, Llama-3-8B FFN-up shape 14336x4096, batch {self.batch}",
                "matrices_per_step": self.copies, "variant": hex(self.variant),
                "tuned": self.tuned is not None,
                "l2": f"inputs larger than L2: {self.copies} distinct weight matrices per rank, "
                      f"{self.copies * self.bytes_per_launch() / 1e6:.0f} MB per step per rank",
                "parallelism": f"tp{self.dist.world} (rows sharded, NCCL all-gather of output slices)" if self.dist.on else "1 GPU"}

    # the CPU oracle on a bounded sample of the same workload
    def cpu_baseline(self, budget_s: float = 12.0):
        from oracle import ref

        ref.build()
        pool = ref.Pool()
        mat = ref.Matrix(ref.Q4_K, self.host_w0, self.rows, self.k, pool)
        ref.matmul(self.host_x, mat, pool=pool)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < budget_s and reps < 2000:
            ref.matmul(self.host_x, mat, pool=pool)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": self.bytes_per_launch() / dt / 1e9, "unit": "GB/s", "cores": pool.threads, "kind": "port",
                "isa": ref.build_info(),
                "sample": f"{reps} multiplies of one {self.rows}x{self.k} Q4_K matrix, batch {self.batch}, "
                          f"{dt * 1e3:.2f} ms each (C++ restatement of the reference's src/ref panel matmul)"}


class DecodeStep:
    """configs[4]: one decode step of a random-init Llama-3-8B-shaped model in Q4_K (32 layers, hidden 4096,
    32 query / 8 KV heads of 128, SwiGLU 14336, RMSNorm, RoPE theta 5e5, vocab 128256 with a Q8_0 head) over
    an f16 KV cache of 8192 positions ~ N(0,1), for `batch` independent sequences. With N ranks the weights
    are row-sharded, attention is sharded by KV head, and output slices are all-gathered over NCCL."""

    name = "decode"
    context = 8192

    def __init__(self, dist: Dist, batch: int = 1, variant: int = 0, layers: int = 32,
                 exchange: str = "peer", attn_variant: int = 0, batched: str = "auto", tune: bool = True, e2e: str = "sample", arena1: bool = False, fuse_combine: bool = True):
        import ctypes as C

        import torch

        from zllm_b200 import abi
        from zllm_b200 import kernels as K
        from zllm_b200 import model as M
        from zllm_b200.plan import DenseConfig, DenseProgram, Shard
        from zllm_b200.torch_util import TorchBuf, nccl_gather

        self.torch, self.K, self.dist, self.batch = torch, K, dist, batch
        self.dev = torch.device("cuda", dist.local)
        torch.cuda.set_device(self.dev)
        self.stream = torch.cuda.Stream(self.dev)
        self.ctx = abi.Context(dist.local, stream=self.stream.cuda_stream)
        self.cfg = DenseConfig(layers=layers, max_ctx=self.context + 64)
        self.shard = Shard(dist.rank, dist.world)
        self.weights, self._keep = M.device_model(self.cfg, torch, self.dev, self.shard)
        self.bufs = []

        def alloc(nbytes):
            b = TorchBuf(torch, self.dev, nbytes)
            self.bufs.append(b)
            return b

        # N ranks exchange output slices either by the kernels themselves (stores into every rank's arena over
        # NVLink, counters instead of collectives) or by NCCL all-gathers between the kernels
        self.exchange = exchange if (dist.on or (arena1 and exchange == "peer")) else "none"
        arena = None
        if self.exchange == "peer":
            def handles(h: bytes):
                got = [None] * dist.world
                dist.dist.all_gather_object(got, h)
                return got

            arena = abi.PeerArena(self.ctx, dist.rank, dist.world, DenseProgram.arena_bytes(self.cfg, batch),
                                  DenseProgram.arena_slots(self.cfg), handles)
        self.prog = DenseProgram(self.ctx, self.cfg, self.weights, batch, alloc, self.shard, arena=arena,
                                 variants={"attn_split": attn_variant} if attn_variant else None,
                                 batched=None if batched == "auto" else batched == "on",
                                 gather=nccl_gather(dist.dist, dist.rank, dist.world) if self.exchange == "nccl" else None)
        self.prog.fuse_combine = self.prog.fuse_combine and fuse_combine
        if arena is not None:
            class _View:  # the arena's logits as a torch tensor (zero copy), for the read-back of the e2e leg
                __cuda_array_interface__ = {"shape": (batch * self.cfg.vocab,), "typestr": "<f4",
                                            "data": (self.prog.logits.ptr, False), "version": 2}

            self.logits_view = torch.as_tensor(_View(), device=self.dev)
        else:
            self.logits_view = self.prog.logits.f32()
        table = alloc(self.cfg.max_ctx * self.cfg.head_dim * 4)
        table.upload(DenseProgram.rope_table(self.cfg))
        self.prog.set_rope_table(table)
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(1234 + dist.rank)
        for il in range(self.cfg.layers):  # the cache before the step: N(0,1) as f16
            for cache in (self.prog.kc[il], self.prog.vc[il]):
                v = cache.t[: cache.nbytes].view(torch.float16)
                v.copy_(torch.randn(v.numel(), device=self.dev, generator=gen, dtype=torch.float32).to(torch.float16))
        rng = np.random.default_rng(99)
        self.tokens = rng.integers(0, self.cfg.vocab, size=batch).astype(np.uint32)
        self.positions = np.full(batch, self.context, dtype=np.uint32)
        self.pinned_tokens = torch.from_numpy(self.tokens.view(np.int32).copy()).pin_memory()
        self.pinned_logits = torch.empty((batch, self.cfg.vocab), dtype=torch.float32).pin_memory()
        self.prog.write_step(self.tokens, self.positions)
        torch.cuda.synchronize()
        # the load-time sweep over the decode multiply's variants (tiles in flight, CTA shape, CTA count) on the
        # model's own weights, as the reference tunes at load (src/tune/tune.zig); steps of up to four sequences
        self.tuned = {}
        if tune and batch <= 4:
            self.tuned = self.prog.sweep()
            torch.cuda.synchronize()
            # ... and the best few of each shape tried inside the replayed step (every rank runs the same trials)
            if self.exchange != "nccl":
                dist.barrier()
                self.tuned = {k: v for k, v in self.prog.refine(self.context + 1, agree=dist.max_each).items() if isinstance(k, tuple)}
                torch.cuda.synchronize()
                dist.barrier()
        self.graph = None
        self.tgraph = None
        self.mv_graph = None
        self.bytes = self.prog.algorithmic_bytes(self.positions)
        # The end-to-end leg draws each sequence's next token on the GPU (the reference's sampler at temperature 0:
        # src/sampler/sampler.zig), so a step costs the host 4 bytes in and 16 bytes out per sequence, not a row of logits.
        self.e2e = e2e
        vocab = self.cfg.vocab
        self.s_block = K.sample_params(vocab, temperature=0.0)
        self.s_params = alloc(C.sizeof(K.Sample)).upload(np.frombuffer(bytes(self.s_block), dtype=np.uint8).copy())
        self.s_bias, self.s_mask = alloc(256), alloc(vocab * 4)
        self.s_counts, self.s_work = alloc(vocab * 4), alloc(vocab * 4)
        self.s_state = [alloc(K.sample_state_words(vocab) * 4) for _ in range(batch)]
        self.s_next = alloc(16 * batch)
        self.s_step = alloc(16).upload(np.array([1, 0, 0, 0], dtype=np.uint32))
        self.pinned_next = torch.empty((batch, 4), dtype=torch.int32).pin_memory()
        torch.cuda.synchronize()

    def _record(self):
        self.prog.record_step(self.context + 1)

    def step(self):
        torch = self.torch
        if self.exchange != "nccl":
            if self.graph is None:
                self.ctx.capture_begin()
                self._record()
                self.graph = self.ctx.capture_end()
            self.ctx.graph_launch(self.graph)
            return
        if self.tgraph is None:
            with torch.cuda.stream(self.stream):
                self._record()  # warm NCCL up outside the capture
                self.stream.synchronize()
                self.tgraph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.tgraph, stream=self.stream):
                    self._record()
        with torch.cuda.stream(self.stream):
            self.tgraph.replay()

    def draw(self):
        """One greedy draw per sequence from the step's logits (one launch each); the tokens land in s_next."""
        vocab, K = self.cfg.vocab, self.K
        for b in range(self.batch):
            logits = (self.logits_view.data_ptr() + 4 * b * vocab, 4 * vocab)
            self.prog.L.sample(self.s_block, self.s_params, logits, self.s_bias, self.s_mask, self.s_counts, self.s_work,
                               self.s_state[b], self.s_next.at(16 * b, 16), self.s_step, steps=[(K.PH_PREP, 0)])

    def e2e_step(self):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            self.prog.tokens.t[: 4 * self.batch].view(torch.int32).copy_(self.pinned_tokens, non_blocking=True)
        self.step()
        if self.e2e == "sample":
            self.draw()
            with torch.cuda.stream(self.stream):
                self.pinned_next.copy_(self.s_next.t[: 16 * self.batch].view(torch.int32).view(self.batch, 4), non_blocking=True)
        else:
            with torch.cuda.stream(self.stream):
                self.pinned_logits.copy_(self.logits_view.view(self.batch, self.cfg.vocab), non_blocking=True)
        self.stream.synchronize()

    def e2e_check(self) -> bool:
        """After an e2e step: the drawn tokens are the logits' largest entries (the first of equals)."""
        if self.e2e != "sample":
            return True
        logits = self.logits_view.view(self.batch, self.cfg.vocab).float().cpu().numpy()
        return bool((self.pinned_next[:, 0].numpy().astype(np.int64) == logits.argmax(axis=1)).all())

    def e2e_bytes(self):
        if self.e2e == "sample":
            return self.tokens.nbytes, self.pinned_next.numel() * 4
        return self.tokens.nbytes, self.pinned_logits.numel() * 4

    def e2e_launches(self) -> int:
        return self.batch if self.e2e == "sample" else 0

    def launches_per_step(self) -> int:
        return self.prog.launches_per_step or (2 + 7 * self.cfg.layers)

    def metric(self):
        return "decode_tokens_per_s", "tokens/s"

    def value(self, seconds_per_step: float) -> float:
        return self.batch / seconds_per_step

    def config(self):
        c = self.cfg
        return {"workload": f"decode step, Llama-3-8B-shaped Q4_K model ({c.layers} layers, hidden {c.hidden}, "
                            f"{c.heads}/{c.kv_heads} heads of {c.head_dim}, FFN {c.ff}, vocab {c.vocab} Q8_0 head), "
                            f"f16 KV cache at {self.context} positions, batch {self.batch}",
                "batch": self.batch, "context": self.context,
                "replay": "CUDA graph of the step's launches",
                "tuned_variants": {f"{t} {n}x{k}": hex(v) for (t, n, k), v in self.tuned.items()},
                "l2": f"inputs larger than L2: a step reads {self.bytes['total'] / 1e9:.2f} GB per rank "
                      f"({self.bytes['weights'] / 1e9:.2f} GB weights + {self.bytes['kv'] / 1e9:.2f} GB KV)",
                "parallelism": ("1 GPU" if not self.dist.on else
                                f"tp{self.dist.world} (rows and KV heads sharded; output slices " +
                                ("pushed into every rank's arena by the kernels' epilogues over NVLink, counters for collectives)"
                                 if self.exchange == "peer" else "all-gathered by NCCL)")),
                "step_bytes": self.bytes["total"]}

    def roofline(self, ms_per_step: float):
        """The dominant kernel (the Q4_K decode multiply): its launches of one step replayed on their own,
        timed with CUDA events, against their algorithmic bytes."""
        torch, K, cfg = self.torch, self.K, self.cfg
        from zllm_b200.plan import layer_weight_shapes

        shapes = layer_weight_shapes(cfg, self.shard)
        p = self.prog
        if self.mv_graph is None:
            # the body multiplies of a step as the step launches them, without the attention between them. On one
            # GPU they hand their vectors on through the exchange slots exactly as in the step (x after wo -> gate|up
            # -> down -> the next layer's Q|K|V); only wo, whose input the attention would push, reads plain memory,
            # and the last down pushes nothing (the head, its consumer, is not part of this list).
            chained = p.arena is not None and self.dist.world == 1   # (a world-of-one exchange, when the program was given an arena)
            self.ctx.capture_begin()
            for il in range(cfg.layers):
                lw = self.weights["layers"][il]
                _, s_xwo, s_act, s_xdown, s_prev = p._slots(il) if chained else (None,) * 5
                if chained and il == cfg.layers - 1:
                    s_xdown = None
                p._matvec(cfg.body_type, p.x, lw["wqkv"], p.qkv, p.qkv_row, cfg.hidden, flags=K.NORM, eps=cfg.eps,
                          norm_w=lw["attn_norm"], wait=s_prev)
                p._matvec(cfg.body_type, p.att, lw["wo"], p.x, p.le, cfg.q_dim, col0=self.shard.rank * p.le,
                          out_stride=cfg.hidden, flags=K.ACCUMULATE, push=s_xwo)
                p._matvec(cfg.body_type, p.x, lw["wgu"], p.act, p.lff, cfg.hidden, col0=self.shard.rank * p.lff,
                          out_stride=cfg.ff, flags=K.NORM | K.SILU_PAIR, eps=cfg.eps, half=p.lff, norm_w=lw["ffn_norm"],
                          wait=s_xwo, push=s_act)
                p._matvec(cfg.body_type, p.act, lw["wdown"], p.x, p.le, cfg.ff, col0=self.shard.rank * p.le,
                          out_stride=cfg.hidden, flags=K.ACCUMULATE, wait=s_act, push=s_xdown)
            if chained:
                p.L.peer_next()
            self.mv_graph = self.ctx.capture_end()
        for _ in range(3):
            self.ctx.graph_launch(self.mv_graph)
        self.stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        e0.record(self.stream)
        for _ in range(reps):
            self.ctx.graph_launch(self.mv_graph)
        e1.record(self.stream)
        self.stream.synchronize()
        multiplies = 4 * cfg.layers
        launches = multiplies
        us = e0.elapsed_time(e1) * 1e3 / (reps * launches)
        wbytes = sum(r * K.row_bytes(cfg.body_type, k) for r, k in shapes.values()) * cfg.layers
        act = 4 * self.batch * cfg.layers * (cfg.hidden * 2 + cfg.q_dim + cfg.ff + p.qkv_row + 2 * p.le + p.lff)
        per_launch = (wbytes + act) / launches
        achieved = per_launch / us / 1e3
        peak, kind = measured_hbm_peak()
        kernel = "matvec_imma<Q4_K> (the 4 body multiplies of each layer, mean over a step)"
        return {"bound": "hbm", "kernel": kernel,
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {kind}",
                "frac_of_8000_nominal": achieved / 8000.0,
                # dram__bytes_read + write of the same four multiplies from an ncu capture of this workload on one GPU
                # (14.26, 9.54, 66.16 and 33.17 MB: profiles/matvec_imma_decode_traffic.md); not captured for sharded
                # or batched runs
                "traffic": (30.78e6 * multiplies / launches) if (self.dist.world == 1 and self.batch == 1) else None,
                "bytes_per_launch": per_launch, "multiplies_per_launch": multiplies / launches,
                "us_per_launch": us, "us_per_multiply": us * launches / multiplies, "launches_per_step": launches,
                "step_hbm_gbs": self.bytes["total"] / (ms_per_step * 1e-3) / 1e9,
                "step_frac": self.bytes["total"] / (ms_per_step * 1e-3) / 1e9 / peak}

    def cpu_baseline(self, budget_s: float = 20.0):
        return cpu_decode_baseline(self.cfg, self.context, budget_s)


def cpu_decode_baseline(cfg, context, budget_s=20.0, sample_layers=2):
    """The CPU oracle (the C++ restatement of the reference's src/ref path) on a bounded sample of the decode
    step: `sample_layers` layers and the head at batch 1, extrapolated to all layers."""
    from oracle import ref
    from zllm_b200 import kernels as K
    from zllm_b200 import synth

    ref.build()
    pool = ref.Pool()
    e, hd = cfg.hidden, cfg.head_dim
    rng = synth.rng_for("cfg5", "cpu")

    def mat(n, k):
        return ref.Matrix(ref.Q4_K, synth.q4_k_weights(rng, n, k), n, k, pool)

    layer = {"attn_norm": np.ones(e, dtype=np.float32), "ffn_norm": np.ones(e, dtype=np.float32),
             "wq": mat(cfg.q_dim, e), "wk": mat(cfg.kv_dim, e), "wv": mat(cfg.kv_dim, e), "wo": mat(e, cfg.q_dim),
             "gate": mat(cfg.ff, e), "up": mat(cfg.ff, e), "down": mat(e, cfg.ff)}
    head = ref.Matrix(ref.Q8_0, synth.q8_0_weights(rng, cfg.vocab, e), cfg.vocab, e, pool)
    kc = rng.normal(size=(context + 1, cfg.kv_heads, hd)).astype(np.float16).view(np.uint16)
    vc = rng.normal(size=(context + 1, cfg.kv_heads, hd)).astype(np.float16).view(np.uint16)
    x = synth.normal_f32(rng, e)
    out_norm = np.ones(e, dtype=np.float32)

    def one_layer(v):
        return ref.dense_decode_layer(layer, v, kc, vc, context, cfg.heads, cfg.kv_heads, hd, cfg.ff, cfg.eps,
                                      cfg.rope_base, K.attention_scale(hd), pool=pool)

    x = one_layer(x)  # warm-up
    t_layers, reps = 0.0, 0
    t0 = time.perf_counter()
    while reps < sample_layers or (time.perf_counter() - t0 < budget_s * 0.6 and reps < 8 * sample_layers):
        t1 = time.perf_counter()
        x = one_layer(x * np.float32(1e-3))
        t_layers += time.perf_counter() - t1
        reps += 1
    t_layer = t_layers / reps
    ref.dense_head(x, out_norm, head, cfg.eps, pool=pool)
    t1 = time.perf_counter()
    ref.dense_head(x, out_norm, head, cfg.eps, pool=pool)
    t_head = time.perf_counter() - t1
    step_s = cfg.layers * t_layer + t_head
    return {"value": 1.0 / step_s, "unit": "tokens/s", "cores": pool.threads, "kind": "port", "isa": ref.build_info(),
            "sample": f"{reps} decode layers ({t_layer * 1e3:.1f} ms each) and one Q8_0 head ({t_head * 1e3:.1f} ms) at "
                      f"batch 1, context {context}, extrapolated to {cfg.layers} layers: {step_s * 1e3:.0f} ms per token "
                      "(C++ restatement of the reference's src/ref forward)"}


class PrefillMatmul:
    """configs[2]: activations bf16 [2048, 4096] ~ N(0,1); weights bf16 [4096, 4096] ~ N(0, 0.02); f32 accumulation
    in tensor memory; bf16 out. The tensor-core prefill rung (tcgen05). With N ranks the weight rows are sharded
    and every rank multiplies the full activations by its rows (no collective in the timed step)."""

    rows, n, k = 2048, 4096, 4096
    name = "prefill_matmul"
    dtype = "bf16"

    def __init__(self, dist: Dist, batch: int = 1, variant: int = 0, **_):
        import torch

        from zllm_b200 import abi
        from zllm_b200 import kernels as K

        self.torch, self.K, self.dist = torch, K, dist
        self.dev = torch.device("cuda", dist.local)
        torch.cuda.set_device(self.dev)
        self.stream = torch.cuda.Stream(self.dev)
        self.ctx = abi.Context(dist.local, stream=self.stream.cuda_stream)
        self.launcher = K.Launcher(self.ctx)
        self.copies = 8                                   # 8 distinct weight matrices: 268 MB > the 126 MB L2
        self.ln = self.n // dist.world
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(4321 + dist.rank)
        self.w = (torch.randn((self.copies, self.ln, self.k), device=self.dev, generator=gen) * 0.02).to(torch.bfloat16)
        self.pinned_x = torch.randn((self.rows, self.k), generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
        self.x = self.pinned_x.to(self.dev)
        self.out = torch.zeros((self.copies, self.rows, self.ln), dtype=torch.bfloat16, device=self.dev)
        self.pinned_out = torch.empty((self.rows, self.ln), dtype=torch.bfloat16).pin_memory()
        self.graph = None
        torch.cuda.synchronize()

    def flops_per_launch(self) -> float:
        return 2.0 * self.rows * self.ln * self.k

    def launches_per_step(self) -> int:
        return self.copies

    def _launch_all(self):
        K = self.K
        for c in range(self.copies):
            self.launcher.matmul("bf16", (self.x.data_ptr(), self.x.numel() * 2), (self.w[c].data_ptr(), self.w[c].numel() * 2),
                                 (self.out[c].data_ptr(), self.out[c].numel() * 2), self.rows, self.ln, self.k,
                                 variant=K.VARIANT_PREFILL_TC, layout=K.X_HALF | K.OUT_HALF)

    def step(self):
        if self.graph is None:
            self.ctx.capture_begin()
            self._launch_all()
            self.graph = self.ctx.capture_end()
        self.ctx.graph_launch(self.graph)

    def e2e_step(self):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            self.x.copy_(self.pinned_x, non_blocking=True)
        self.step()
        with torch.cuda.stream(self.stream):
            self.pinned_out.copy_(self.out[self.copies - 1], non_blocking=True)
        self.stream.synchronize()

    def e2e_bytes(self):
        return self.pinned_x.numel() * 2, self.pinned_out.numel() * 2

    def roofline(self, ms_per_step: float):
        peak, kind = measured_tensor_peak()
        us = ms_per_step * 1e3 / self.launches_per_step()
        achieved = self.flops_per_launch() / us / 1e6
        return {"bound": "tensor", "kernel": "matmul_tc_kernel<bf16>", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "peak_kind": f"of {kind}", "traffic": None, "flops_per_launch": self.flops_per_launch(),
                "us_per_launch": us}

    def metric(self):
        return "prefill_matmul_tflops", "TFLOP/s"

    def value(self, seconds_per_step: float) -> float:
        return self.flops_per_launch() * self.copies * self.dist.world / seconds_per_step / 1e12

    def config(self):
        return {"workload": f"BF16 prefill matmul, {self.rows} tokens x {self.n} x {self.k}, bf16 in/out, f32 accumulate (tcgen05)",
                "matrices_per_step": self.copies,
                "l2": f"inputs larger than L2: {self.copies} distinct weight matrices, {self.copies * self.ln * self.k * 2 / 1e6:.0f} MB per step per rank",
                "parallelism": f"tp{self.dist.world} (weight rows sharded, no collective in the step)" if self.dist.on else "1 GPU"}

    def cpu_baseline(self, budget_s: float = 12.0):
        from oracle import ref
        from zllm_b200 import synth

        ref.build()
        pool = ref.Pool()
        rng = synth.rng_for("cfg3", "cpu")
        rows = 64                                          # a bounded sample: 64 of the 2048 tokens
        mat = ref.Matrix(ref.BF16, synth.bf16_weights(rng, self.n, self.k), self.n, self.k, pool)
        x = ref.round_like_llama(ref.BF16, synth.normal_f32(rng, rows, self.k)).reshape(rows, self.k)
        ref.matmul(x, mat, pool=pool)
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < budget_s and reps < 200:
            ref.matmul(x, mat, pool=pool)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": 2.0 * rows * self.n * self.k / dt / 1e12, "unit": "TFLOP/s", "cores": pool.threads, "kind": "port",
                "isa": ref.build_info(),
                "sample": f"{reps} multiplies of {rows} tokens x {self.n} x {self.k} (bf16 weights, f32 accumulate), {dt * 1e3:.1f} ms each "
                          "(C++ restatement of the reference's src/ref panel matmul)"}


class DeltaPrefill:
    """configs[3], prefill: one Gated DeltaNet layer, batch 1, 4096 tokens, 16 heads of 128; q, k (L2-normalised)
    and v hold bf16 values; beta = sigmoid(N(0,1)); log-decay = -softplus(N(0,1)); f32 state from zero. The chunked
    form (chunk 64). With N ranks the heads are sharded (no collective: heads are independent)."""

    tokens, heads, d = 4096, 16, 128
    name = "deltanet_prefill"
    dtype = "f32"

    def __init__(self, dist: Dist, batch: int = 1, variant: int = 0, **_):
        import torch

        from zllm_b200 import abi, synth
        from zllm_b200 import kernels as K

        self.torch, self.K, self.dist = torch, K, dist
        self.dev = torch.device("cuda", dist.local)
        torch.cuda.set_device(self.dev)
        self.stream = torch.cuda.Stream(self.dev)
        self.ctx = abi.Context(dist.local, stream=self.stream.cuda_stream)
        self.launcher = K.Launcher(self.ctx)
        self.recurrent = variant == 1                     # --variant 1: the serial kernel, for comparison
        self.f32_form = variant == 2                      # --variant 2: the chunked form in f32 on the CUDA cores
        self.lh = self.heads // dist.world
        self.sets = 2                                     # two input sets alternate: 2 x 133 MB > the 126 MB L2
        self.cd = 3 * self.lh * self.d
        self.conv, self.g, self.beta = [], [], []
        for i in range(self.sets):
            conv, g, beta = synth.deltanet_inputs(synth.rng_for("cfg4", f"bench{dist.rank}-{i}"), self.tokens, self.lh, self.lh, self.d)
            self.conv.append(torch.from_numpy(conv).pin_memory())
            self.g.append(torch.from_numpy(g).to(self.dev))
            self.beta.append(torch.from_numpy(beta).to(self.dev))
        self.dconv = [c.to(self.dev) for c in self.conv]
        self.state = torch.zeros((self.lh, self.d, self.d), dtype=torch.float32, device=self.dev)
        self.out = [torch.zeros((self.tokens, self.lh * self.d), dtype=torch.float32, device=self.dev) for _ in range(self.sets)]
        self.pinned_out = torch.empty((self.tokens, self.lh * self.d), dtype=torch.float32).pin_memory()
        self.step_buf = torch.tensor([self.tokens, 0, 0, 0], dtype=torch.int32, device=self.dev)
        self.turn = 0
        torch.cuda.synchronize()

    def launches_per_step(self) -> int:
        return 1 if self.recurrent else 3

    def _buf(self, t):
        return (t.data_ptr(), t.numel() * t.element_size())

    def step(self):
        K, i = self.K, self.turn % self.sets
        self.turn += 1
        with self.torch.cuda.stream(self.stream):
            self.state.zero_()
        p = K.DeltaRule(self.lh, self.lh, self.d, self.cd, 1, self.cd, 0)
        self.launcher.delta_rule(p, self._buf(self.dconv[i]), self._buf(self.g[i]), self._buf(self.beta[i]), self._buf(self.state),
                                 self._buf(self.out[i]), self._buf(self.step_buf),
                                 chunked_tokens=None if self.recurrent else self.tokens,
                                 chunk_variant=K.VARIANT_DELTA_CHUNK64_F32 if self.f32_form else K.VARIANT_DELTA_CHUNK64)

    def e2e_step(self):
        torch, i = self.torch, self.turn % self.sets
        with torch.cuda.stream(self.stream):
            self.dconv[i].copy_(self.conv[i], non_blocking=True)
        self.step()
        with torch.cuda.stream(self.stream):
            self.pinned_out.copy_(self.out[i], non_blocking=True)
        self.stream.synchronize()

    def e2e_bytes(self):
        return self.conv[0].numel() * 4, self.pinned_out.numel() * 4

    def bytes_per_step(self) -> float:
        # q, k, v in, o out (f32 here), g and beta, the state in and out
        return 4.0 * self.tokens * (self.cd + self.lh * self.d + 2 * self.lh) + 2 * 4.0 * self.lh * self.d * self.d

    def flops_per_step(self) -> float:
        c, d = 64, self.d
        return (6.0 * c * d * d + 8.0 * c * c * d) * (self.tokens / c) * self.lh

    def roofline(self, ms_per_step: float):
        peak, kind = measured_hbm_peak()
        achieved = self.bytes_per_step() / (ms_per_step * 1e-3) / 1e9
        kernel = "delta_rule_kernel" if self.recurrent else ("delta_chunk_scan + delta_chunk_prep (f32, CUDA cores)" if self.f32_form
                                                           else "delta_chunk_scan_tc (tcgen05, bf16 x 2 terms) + delta_chunk_prep_tc")
        return {"bound": "hbm", "kernel": kernel,
                "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {kind}",
                "traffic": None, "bytes_per_launch": self.bytes_per_step(),
                "algorithmic_tflops": self.flops_per_step() / (ms_per_step * 1e-3) / 1e12,
                "us_per_chunk_step": ms_per_step * 1e3 / (self.tokens / 64),
                "note": "neither roofline binds: a head's 64 chunks are a serial chain; the chunk step's latency is the figure to lower"}

    def metric(self):
        return "deltanet_prefill_tokens_per_s", "tokens/s"

    def value(self, seconds_per_step: float) -> float:
        return self.tokens / seconds_per_step

    def config(self):
        return {"workload": f"Gated DeltaNet layer prefill, batch 1, {self.tokens} tokens, {self.heads} heads of {self.d}, "
                            + ("recurrent form" if self.recurrent else "chunked form (chunk 64), f32 on the CUDA cores" if self.f32_form
                               else "chunked form (chunk 64) on the tensor cores"),
                "l2": f"inputs larger than L2: {self.sets} input sets alternate, {self.bytes_per_step() / 1e6:.0f} MB each",
                "parallelism": f"heads sharded over {self.dist.world} ranks, no collective" if self.dist.on else "1 GPU"}

    def cpu_baseline(self, budget_s: float = 12.0):
        from oracle import ref
        from zllm_b200 import synth

        ref.build()
        sample = 512                                       # a bounded sample: the first 512 of the 4096 tokens
        conv, g, beta = synth.deltanet_inputs(synth.rng_for("cfg4", "cpu"), sample, self.heads, self.heads, self.d)
        zero = np.zeros((self.heads, self.d, self.d), dtype=np.float32)
        ref.delta_rule(zero, conv, g, beta, sample, self.heads, self.heads, self.d)
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < budget_s and reps < 50:
            ref.delta_rule(zero, conv, g, beta, sample, self.heads, self.heads, self.d)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": sample / dt, "unit": "tokens/s", "cores": min(ref.default_pool().threads, self.heads), "kind": "port", "isa": ref.build_info(),
                "sample": f"{reps} runs of the first {sample} tokens, all {self.heads} heads, {dt * 1e3:.1f} ms each "
                          "(C++ restatement of the reference's src/ref recurHead, one head per task)"}


class DeltaDecode:
    """configs[3], recurrent decode: one token of a Gated DeltaNet layer (16 heads of 128, q / k L2-normalised bf16
    values, v bf16 values, beta = sigmoid(N(0,1)), log-decay = -softplus(N(0,1))) on a seeded f32 state. A step is a
    CUDA graph over `layers` independent layer states (as many DeltaNet layers of a model, 1 MiB of state each,
    together above the L2 size), each updated by one delta_rule launch. With N ranks the value heads (and their key
    heads) are sharded; heads are independent, so no collective."""

    heads, d, layers = 16, 128, 160
    name = "deltanet_decode"
    dtype = "f32"
    scaling = "strong"

    def __init__(self, dist: Dist, batch: int = 1, variant: int = 0, **_):
        import torch

        from zllm_b200 import abi, synth
        from zllm_b200 import kernels as K

        self.torch, self.K, self.dist = torch, K, dist
        self.dev = torch.device("cuda", dist.local)
        torch.cuda.set_device(self.dev)
        self.stream = torch.cuda.Stream(self.dev)
        self.ctx = abi.Context(dist.local, stream=self.stream.cuda_stream)
        self.launcher = K.Launcher(self.ctx)
        self.lh = self.heads // dist.world
        self.cd = 3 * self.lh * self.d
        gen = torch.Generator(device=self.dev)
        gen.manual_seed(99 + dist.rank)
        # the state a 64-token prefix leaves is of order one; a seeded random state of that size stands in per layer
        self.state = (torch.randn((self.layers, self.lh, self.d, self.d), device=self.dev, generator=gen) * 0.1).float()
        conv, g, beta = synth.deltanet_inputs(synth.rng_for("cfg4", f"decode-bench{dist.rank}"), self.layers, self.lh, self.lh, self.d)
        self.pinned_conv = torch.from_numpy(conv).pin_memory()          # one token's q | k | v per layer
        self.conv = self.pinned_conv.to(self.dev)
        self.g = torch.from_numpy(g).to(self.dev)
        self.beta = torch.from_numpy(beta).to(self.dev)
        self.out = torch.zeros((self.layers, self.lh * self.d), dtype=torch.float32, device=self.dev)
        self.pinned_out = torch.empty((self.layers, self.lh * self.d), dtype=torch.float32).pin_memory()
        self.step_buf = torch.tensor([1, 64, 0, 0], dtype=torch.int32, device=self.dev)
        self.graph = None
        torch.cuda.synchronize()

    def launches_per_step(self) -> int:
        return self.layers

    def _buf(self, t):
        return (t.data_ptr(), t.numel() * t.element_size())

    def step(self):
        K = self.K
        if self.graph is None:
            self.ctx.capture_begin()
            p = K.DeltaRule(self.lh, self.lh, self.d, self.cd, 1, self.cd, 0)
            for il in range(self.layers):
                self.launcher.delta_rule(p, self._buf(self.conv[il]), self._buf(self.g[il]), self._buf(self.beta[il]),
                                         self._buf(self.state[il]), self._buf(self.out[il]), self._buf(self.step_buf))
            self.graph = self.ctx.capture_end()
        self.ctx.graph_launch(self.graph)

    def e2e_step(self):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            self.conv.copy_(self.pinned_conv, non_blocking=True)
        self.step()
        with torch.cuda.stream(self.stream):
            self.pinned_out.copy_(self.out, non_blocking=True)
        self.stream.synchronize()

    def e2e_bytes(self):
        return self.pinned_conv.numel() * 4, self.pinned_out.numel() * 4

    def bytes_per_launch(self) -> float:
        # the state in and out, q | k | v, g, beta in, o out
        return 2 * 4.0 * self.lh * self.d * self.d + 4.0 * (self.cd + self.lh * self.d + 2 * self.lh)

    def roofline(self, ms_per_step: float):
        peak, kind = measured_hbm_peak()
        us = ms_per_step * 1e3 / self.layers
        achieved = self.bytes_per_launch() / us / 1e3
        return {"bound": "hbm", "kernel": "delta_rule_kernel (recurrent form, one token)", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {kind}", "traffic": None, "bytes_per_launch": self.bytes_per_launch(),
                "us_per_launch": us,
                "note": "2.1 MB per launch is a third of a microsecond at the roofline: the launch's latency is what is measured"}

    def metric(self):
        return "deltanet_decode_layer_tokens_per_s", "layer-tokens/s"

    def value(self, seconds_per_step: float) -> float:
        return self.layers / seconds_per_step

    def config(self):
        return {"workload": f"Gated DeltaNet recurrent decode, 1 token on a seeded state, {self.heads} heads of {self.d}; "
                            f"{self.layers} independent layer states per step",
                "l2": f"inputs larger than L2: {self.layers} states of {self.lh * self.d * self.d * 4 / 1e6:.2f} MB per rank per step",
                "parallelism": f"value heads sharded over {self.dist.world} ranks, no collective" if self.dist.on else "1 GPU"}

    def cpu_baseline(self, budget_s: float = 10.0):
        from oracle import ref
        from zllm_b200 import synth

        ref.build()
        rng = synth.rng_for("cfg4", "cpu-decode")
        conv, g, beta = synth.deltanet_inputs(rng, 1, self.heads, self.heads, self.d)
        state = (rng.normal(size=(self.heads, self.d, self.d)) * 0.1).astype(np.float32)
        ref.delta_rule(state, conv, g, beta, 1, self.heads, self.heads, self.d)
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < budget_s and reps < 20000:
            ref.delta_rule(state, conv, g, beta, 1, self.heads, self.heads, self.d)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": 1.0 / dt, "unit": "layer-tokens/s", "cores": min(ref.default_pool().threads, self.heads), "kind": "port",
                "isa": ref.build_info(),
                "sample": f"{reps} single-token updates of one layer's state ({self.heads} heads), {dt * 1e6:.0f} us each "
                          "(C++ restatement of the reference's src/ref recurHead, one head per task)"}


class QuantPrefill:
    """The quantised prefill multiply (the reference's prefill path for K-quant models: quantize_q8 + matmul_q4_k):
    2048 tokens x the Llama-3-8B FFN-up matrix (14336 x 4096, Q4_K); activations f32 ~ N(0,1) rounded to Q8_K blocks
    inside the timed step. With N ranks the weight rows are sharded (no collective in the step)."""

    rows, n, k = 2048, 14336, 4096
    name = "prefill_q4_k"
    dtype = "u4 x s8 integer products (exact), f32 sums and scales"

    def __init__(self, dist: Dist, batch: int = 1, variant: int = 0, **_):
        import torch

        from zllm_b200 import abi, synth
        from zllm_b200 import kernels as K

        self.torch, self.K, self.dist = torch, K, dist
        self.dev = torch.device("cuda", dist.local)
        torch.cuda.set_device(self.dev)
        self.stream = torch.cuda.Stream(self.dev)
        self.ctx = abi.Context(dist.local, stream=self.stream.cuda_stream)
        self.launcher = K.Launcher(self.ctx)
        # --variant 0: the tcgen05 rung (0xfffc0000); --variant 1: the integer-dot identity on mma.sync
        self.rung = 0 if variant == 1 else K.VARIANT_PREFILL_TC
        self.copies = 4                                  # 4 distinct matrices: 132 MB of weights + 235 MB of outputs per step
        self.ln = self.n // dist.world
        rb = K.row_bytes("q4_k", self.k)
        one = torch.from_numpy(synth.q4_k_weights(synth.rng_for("cfg2", f"w-rank{dist.rank}"), self.ln, self.k).reshape(-1)).to(self.dev)
        self.w = torch.stack([torch.roll(one.view(self.ln, rb), shifts=c, dims=0).reshape(-1) for c in range(self.copies)])
        self.pinned_x = torch.randn((self.rows, self.k), generator=torch.Generator().manual_seed(11)).pin_memory()
        self.x = self.pinned_x.to(self.dev)
        self.qx = torch.zeros((self.rows, self.k), dtype=torch.int8, device=self.dev)
        self.dx = torch.zeros((self.rows, self.k // 256), dtype=torch.float32, device=self.dev)
        self.out = torch.zeros((self.copies, self.rows, self.ln), dtype=torch.float32, device=self.dev)
        self.pinned_out = torch.empty((self.rows, self.ln), dtype=torch.float32).pin_memory()
        self.graph = None
        torch.cuda.synchronize()

    def _buf(self, t):
        return (t.data_ptr(), t.numel() * t.element_size())

    def flops_per_launch(self) -> float:
        return 2.0 * self.rows * self.ln * self.k

    def launches_per_step(self) -> int:
        return 1 + self.copies * (3 if self.rung else 1)  # the rung: columns, scale-table clear, multiply

    def _launch_all(self):
        self.launcher.quantize_q8(self._buf(self.x), self._buf(self.qx), self._buf(self.dx), self.rows, self.k, 256)
        for c in range(self.copies):
            self.launcher.matmul_quant("q4_k", self._buf(self.qx), self._buf(self.w[c]), self._buf(self.out[c]), self._buf(self.dx),
                                       self.rows, self.ln, self.k, variant=self.rung)

    def step(self):
        if self.graph is None:
            self.ctx.capture_begin()
            self._launch_all()
            self.graph = self.ctx.capture_end()
        self.ctx.graph_launch(self.graph)

    def e2e_step(self):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            self.x.copy_(self.pinned_x, non_blocking=True)
        self.step()
        with torch.cuda.stream(self.stream):
            self.pinned_out.copy_(self.out[self.copies - 1], non_blocking=True)
        self.stream.synchronize()

    def e2e_bytes(self):
        return self.pinned_x.numel() * 4, self.pinned_out.numel() * 4

    def roofline(self, ms_per_step: float):
        peak, kind = measured_tensor_peak()
        us = ms_per_step * 1e3 / self.copies  # the one quantize_q8 of a step is counted into its multiplies
        achieved = self.flops_per_launch() / us / 1e6
        kernel = ("qgemm_q4k_kernel<128> (tcgen05 kind::f16 on f16 integers, accumulators in tensor memory)" if self.rung
                  else "matmul_quant_kernel<Q4_K> (mma.sync s8, unit scales on the CUDA cores)")
        return {"bound": "tensor", "kernel": kernel, "achieved": achieved,
                "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_kind": f"of {kind} (the dense bf16 cuBLAS figure)", "traffic": None,
                "flops_per_launch": self.flops_per_launch(), "us_per_launch": us}

    def metric(self):
        return "prefill_q4_k_matmul_tflops", "TFLOP/s"

    def value(self, seconds_per_step: float) -> float:
        return self.flops_per_launch() * self.copies * self.dist.world / seconds_per_step / 1e12

    def config(self):
        return {"workload": f"Q4_K prefill matmul, {self.rows} tokens x {self.n} x {self.k}, Q8_K-rounded activations (quantize_q8 in the step)",
                "rung": "tcgen05 (variant 0xfffc0000)" if self.rung else "integer dot on mma.sync (variant 0)",
                "matrices_per_step": self.copies,
                "l2": f"inputs larger than L2: {self.copies} weight matrices and outputs, {self.copies * (self.ln * self.k * 9 // 16 + self.rows * self.ln * 4) / 1e6:.0f} MB per step per rank",
                "parallelism": f"tp{self.dist.world} (weight rows sharded, no collective in the step)" if self.dist.on else "1 GPU"}

    def cpu_baseline(self, budget_s: float = 12.0):
        from oracle import ref
        from zllm_b200 import synth

        ref.build()
        pool = ref.Pool()
        rng = synth.rng_for("cfg2", "cpu-prefill")
        rows, n = 32, 2048                                  # a bounded sample: 32 tokens x 2048 of the 14336 rows
        mat = ref.Matrix(ref.Q4_K, synth.q4_k_weights(rng, n, self.k), n, self.k, pool)
        x = synth.normal_f32(rng, rows, self.k)
        ref.matmul(x, mat, act=True, pool=pool)
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < budget_s and reps < 200:
            ref.matmul(x, mat, act=True, pool=pool)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        return {"value": 2.0 * rows * n * self.k / dt / 1e12, "unit": "TFLOP/s", "cores": pool.threads, "kind": "port", "isa": ref.build_info(),
                "sample": f"{reps} multiplies of {rows} tokens x {n} x {self.k} (roundLikeLlama + panel matmul), {dt * 1e3:.1f} ms each "
                          "(C++ restatement of the reference's src/ref)"}


WORKLOADS = {"matvec_q4_k": MatvecQ4K, "decode": DecodeStep, "prefill_matmul": PrefillMatmul, "deltanet_prefill": DeltaPrefill,
             "deltanet_decode": DeltaDecode, "prefill_q4_k": QuantPrefill}



# ------------------------------------------------------------------ arms

def tp_parity(dist, args):
    """N > 1 ranks, outside any timed region: ONE random model (2 layers, the benchmark's widths, its Q8_0 head)
    run sharded over all ranks with the step's exchange, and unsharded on rank 0; the logits are compared on rank 0.
    Returns {"max_rel_l2", "argmax_equal", "bitwise", ...} on rank 0, None elsewhere."""
    import torch

    from zllm_b200 import abi
    from zllm_b200 import model as M
    from zllm_b200.plan import DenseConfig, DenseProgram, Shard
    from zllm_b200.torch_util import TorchBuf, nccl_gather

    dev = torch.device("cuda", dist.local)
    torch.cuda.set_device(dev)
    stream = torch.cuda.Stream(dev)
    ctx = abi.Context(dist.local, stream=stream.cuda_stream)
    batch, context, layers = min(args.batch, 4), 1024, 2
    cfg = DenseConfig(layers=layers, max_ctx=context + 64)
    full = M.device_full_model(cfg, torch, dev, seed=4242)
    bufs = []

    def alloc(nbytes):
        b = TorchBuf(torch, dev, nbytes)
        bufs.append(b)
        return b

    def program(shard, arena=None, gather=None):
        weights, keep = M.device_shard(full, cfg, torch, shard)
        prog = DenseProgram(ctx, cfg, weights, batch, alloc, shard, arena=arena, gather=gather)
        table = alloc(cfg.max_ctx * cfg.head_dim * 4)
        table.upload(DenseProgram.rope_table(cfg))
        prog.set_rope_table(table)
        gen = torch.Generator(device=dev)
        gen.manual_seed(777)   # the same cache on every rank; a rank keeps its KV heads
        g0, g1 = shard.kv_heads(cfg)
        for il in range(cfg.layers):
            for cache in (prog.kc[il], prog.vc[il]):
                whole = torch.randn((batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim), device=dev, generator=gen).to(torch.float16)
                mine = whole[:, :, g0:g1, :].contiguous().view(-1)
                cache.t[: mine.numel() * 2].view(torch.float16).copy_(mine)
        prog.write_step(np.arange(batch, dtype=np.uint32) * 1009 % cfg.vocab + 17, np.full(batch, context, dtype=np.uint32))
        return prog, keep

    shard = Shard(dist.rank, dist.world)
    arena, gather = None, None
    if args.exchange == "peer":
        def handles(h: bytes):
            got = [None] * dist.world
            dist.dist.all_gather_object(got, h)
            return got

        arena = abi.PeerArena(ctx, dist.rank, dist.world, DenseProgram.arena_bytes(cfg, batch), DenseProgram.arena_slots(cfg), handles)
    else:
        gather = nccl_gather(dist.dist, dist.rank, dist.world)
    sharded, keep_s = program(shard, arena=arena, gather=gather)
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.stream(stream):
        sharded.record_step(context + 1)
    ctx.sync()
    dist.barrier()
    out = None
    if dist.rank == 0:
        got = sharded.logits.download(np.float32)[: batch * cfg.vocab].copy()
        whole, keep_w = program(Shard())
        with torch.cuda.stream(stream):
            whole.record_step(context + 1)
        ctx.sync()
        want = whole.logits.download(np.float32)[: batch * cfg.vocab]
        got, want = got.reshape(batch, cfg.vocab), want.reshape(batch, cfg.vocab)
        rel = float(max(np.linalg.norm(got[b] - want[b]) / np.linalg.norm(want[b]) for b in range(batch)))
        out = {"max_rel_l2": rel, "argmax_equal": bool((got.argmax(axis=1) == want.argmax(axis=1)).all()),
               "bitwise": bool(np.array_equal(got.view(np.uint32), want.view(np.uint32))),
               "what": f"{layers} layers of the benchmark's widths + its Q8_0 head, one random model sharded over {dist.world} ranks "
                       f"against the same model on rank 0 alone; batch {batch}, context {context}; exchange {args.exchange}"}
    dist.barrier()
    return out


def run_cuda(args):
    import torch

    dist = Dist(args.gpus)
    parity = tp_parity(dist, args) if (dist.on and args.workload == "decode") else None
    kw = {"batch": args.batch, "variant": int(args.variant, 0)}
    if args.workload == "matvec_q4_k":
        kw["tune"] = not args.no_tune
    if args.workload == "decode":
        kw["exchange"] = args.exchange
        kw["attn_variant"] = args.attn_variant
        kw["batched"] = args.batched
        kw["tune"] = not args.no_tune
        kw["e2e"] = args.e2e
        kw["arena1"] = args.arena
        kw["fuse_combine"] = not args.no_fuse_combine
        if args.layers:
            kw["layers"] = args.layers
    wl = WORKLOADS[args.workload](dist, **kw)
    torch.cuda.set_device(dist.local)
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        wl.step()
    wl.stream.synchronize()
    sampler = ClockSampler(dist.local)
    if dist.rank == 0:
        sampler.start()
    # ---- device-timed region: inputs resident in HBM
    dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(wl.stream)
    for _ in range(args.steps):
        wl.step()
    ev1.record(wl.stream)
    wl.stream.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    ms = dist.max(ev0.elapsed_time(ev1))
    # ---- end-to-end region: host buffers, copies inside
    for _ in range(2):
        wl.e2e_step()
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        wl.e2e_step()
    torch.cuda.synchronize()
    e2e_s = dist.max(time.perf_counter() - t0)
    e2e_ok = wl.e2e_check() if hasattr(wl, "e2e_check") else True
    clocks = sampler.stop() if dist.rank == 0 else {}
    sec_per_step = ms / 1e3 / args.steps
    metric, unit = wl.metric()
    h2d, d2h = wl.e2e_bytes()
    line = {
        "metric": metric, "value": wl.value(sec_per_step), "unit": unit, "n_gpus": dist.world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": getattr(wl, "scaling", "strong"), "vs_baseline": None, "dtype": getattr(wl, "dtype", "f32"), "data": "synthetic", "config": wl.config(),
        "clocks": clocks,
        "e2e": {"value": wl.value(e2e_s / args.steps), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                **({"result": "the next token of every sequence, drawn by the GPU sampler at temperature 0; equal to the logits' argmax: "
                              + str(e2e_ok), "launches_per_step": wl.launches_per_step() + wl.e2e_launches()}
                   if getattr(wl, "e2e", None) == "sample" else {})},
        "gpu_launches": wl.launches_per_step() * args.steps,
        "roofline": wl.roofline(ms / args.steps),
    }
    if dist.rank == 0 and dist.world == 1 and not args.no_cpu:
        line["cpu_baseline"] = wl.cpu_baseline()
    failed = not e2e_ok
    if parity is not None:
        line["tp_parity"] = parity
        failed = failed or not (parity["max_rel_l2"] <= 1e-4 and parity["argmax_equal"])
    if dist.rank == 0:
        print(json.dumps(line), flush=True)
        if not e2e_ok:
            print("bench: a drawn token is not its logits' largest entry", file=sys.stderr)
        elif failed:
            print(f"bench: the sharded step differs from the unsharded one: {parity}", file=sys.stderr)
    if dist.on:
        # Leave without tearing NCCL down: captured graphs still hold its kernels, and a teardown that
        # waits on them has hung here. Every rank is past its last collective.
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1 if failed else 0)
    dist.close()
    if failed:
        sys.exit(1)


def run_reference(args):
    """The reference's own CPU implementation of the path (its C++ restatement), all host cores. Each
    step is a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref
    from zllm_b200 import synth

    ref.build()
    if args.workload == "decode":
        from zllm_b200.plan import DenseConfig

        cfg = DenseConfig(layers=args.layers or 32)
        vals = []
        t0 = time.perf_counter()
        base = None
        for i in range(args.warmup + args.steps):
            base = cpu_decode_baseline(cfg, DecodeStep.context, budget_s=4.0, sample_layers=1)
            if i >= args.warmup:
                vals.append(base["value"])
        dt = time.perf_counter() - t0
        value = float(np.mean(vals))
        base["value"] = value
        print(json.dumps({
            "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / value, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"decode step, Llama-3-8B-shaped Q4_K model, f16 KV cache at {DecodeStep.context} "
                                   "positions, batch 1 (extrapolated from sampled layers and one head per step: see cpu_baseline.sample; "
                                   "the C++ port of the reference's src/ref, not its Zig binary)", "batch": 1, "context": DecodeStep.context,
                       "wall_s": dt},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }), flush=True)
        return
    if args.workload == "prefill_matmul":
        wl = PrefillMatmul.__new__(PrefillMatmul)  # shapes only; nothing on a GPU
        vals, base = [], None
        for i in range(args.warmup + args.steps):
            base = wl.cpu_baseline(budget_s=3.0)
            if i >= args.warmup:
                vals.append(base["value"])
        value = float(np.mean(vals))
        base["value"] = value
        print(json.dumps({
            "impl": "reference", "metric": "prefill_matmul_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 8 * 2.0 * wl.rows * wl.n * wl.k / value / 1e9,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"BF16 prefill matmul, {wl.rows} tokens x {wl.n} x {wl.k} (a 64-token sample per step)"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }), flush=True)
        return
    if args.workload in ("deltanet_prefill", "deltanet_decode"):
        cls = WORKLOADS[args.workload]
        wl = cls.__new__(cls)  # shapes only; nothing on a GPU
        vals, base = [], None
        t0 = time.perf_counter()
        for i in range(args.warmup + args.steps):
            base = wl.cpu_baseline(budget_s=3.0)
            if i >= args.warmup:
                vals.append(base["value"])
        value = float(np.mean(vals))
        base["value"] = value
        metric, unit = wl.metric()
        print(json.dumps({
            "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": (time.perf_counter() - t0) / (args.warmup + args.steps) * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"Gated DeltaNet, {cls.heads} heads of {cls.d}: " + base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }), flush=True)
        return
    if args.workload == "prefill_q4_k":
        wl = QuantPrefill.__new__(QuantPrefill)  # shapes only; nothing on a GPU
        wl.k = QuantPrefill.k
        vals, base = [], None
        for i in range(args.warmup + args.steps):
            base = wl.cpu_baseline(budget_s=3.0)
            if i >= args.warmup:
                vals.append(base["value"])
        value = float(np.mean(vals))
        base["value"] = value
        print(json.dumps({
            "impl": "reference", "metric": "prefill_q4_k_matmul_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 4 * 2.0 * wl.rows * wl.n * wl.k / value / 1e9,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": QuantPrefill.dtype, "data": "synthetic",
            "config": {"workload": f"Q4_K prefill matmul, {wl.rows} tokens x {wl.n} x {wl.k}, Q8_K-rounded activations "
                                   "(a 32-token x 2048-row sample per step)"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }), flush=True)
        return
    n, k, batch = MatvecQ4K.n, MatvecQ4K.k, 1
    pool = ref.Pool()
    raw = synth.q4_k_weights(synth.rng_for("cfg2", "w-rank0"), n, k)
    x = synth.normal_f32(synth.rng_for("cfg2", f"x{batch}"), batch, k)
    mat = ref.Matrix(ref.Q4_K, raw, n, k, pool)
    bytes_per = n * (k // 256) * 144 + 4 * batch * k + 4 * batch * n
    reps_per_step = 8
    for _ in range(max(1, args.warmup)):
        ref.matmul(x, mat, pool=pool)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(reps_per_step):
            ref.matmul(x, mat, pool=pool)
    dt = time.perf_counter() - t0
    value = bytes_per * reps_per_step * args.steps / dt / 1e9
    sample = f"{reps_per_step} multiplies per step of one {n}x{k} Q4_K matrix, batch {batch}"
    print(json.dumps({
        "impl": "reference", "metric": "q4_k_matvec_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"Q4_K matvec, Llama-3-8B FFN-up shape {n}x{k}, batch {batch}", "matrices_per_step": reps_per_step},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": pool.threads, "kind": "port", "isa": ref.build_info(), "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS))
    ap.add_argument("--layers", type=int, default=0, help="decode: layers of the model (default 32)")
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--variant", default="0", help="matvec variant word (see include/zllm_cuda.h)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--batched", default="auto", choices=["auto", "on", "off"],
                    help="decode: Q4_K multiplies in one pass for all sequences (tcgen05 family; auto = for 5..64 sequences on one GPU)")
    ap.add_argument("--arena", action="store_true",
                    help="decode on one GPU: the vectors between the kernels go through the tagged slots of a world-of-one exchange, "
                         "and the output projection merges the attention's partials itself (one launch fewer per layer)")
    ap.add_argument("--no-fuse-combine", action="store_true",
                    help="decode with the peer exchange: attn_combine as its own launch instead of the output projection's first phase")
    ap.add_argument("--e2e", default="sample", choices=["sample", "logits"],
                    help="decode, end-to-end leg: the next token drawn on the GPU and read back (16 bytes a sequence), or the logits read back")
    ap.add_argument("--no-tune", action="store_true", help="decode: skip the load-time sweep over the multiply's variants")
    ap.add_argument("--attn-variant", type=int, default=0, help="decode: form of attn_split's fast path (0 default, 1-4: k_attn.cu)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="decode on N > 1 GPUs: slices pushed by the kernels over peer memory, or NCCL all-gathers")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
