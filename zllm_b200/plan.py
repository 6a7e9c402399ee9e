"""The decode-step program of a Llama-shaped dense model: the host-side mirror of the reference's plan for
dense models (src/plan/qwen35.zig:218-280 upload, :451-692 build, :766-805 recordStep,
LayerBuilder.attention :989-1036, ffn :1039-1052), driving the CUDA backend.

Per layer the reference records seven dispatches, and so does this program:
  1. matvec  Wq|Wk|Wv  with the RMSNorm prologue          (plan/qwen35.zig:1006)
  2. rope_append                                           (:1008-1022)
  3. attn_split   4. attn_combine                          (:1023-1034)
  5. matvec  Wo, ACCUMULATE into the residual stream       (:1034)
  6. matvec  gate|up with NORM + SILU_PAIR                 (:1048)
  7. matvec  Wdown, ACCUMULATE                             (:1049)
then the output norm fused into the LM-head matvec (:609), after one embed_* at the front (:549-551).
Weights that share an input are stacked by rows (Q|K|V, gate|up: :255-262).

Two things go beyond the reference, which runs one sequence on one GPU:
  * a batch of B independent sequences, each with its own KV cache and position (rows of the step are
    sequences; attention and rope_append take the per-sequence cache stride and positions);
  * tensor parallelism over W ranks: every weight matrix is sharded by rows per part (query heads and
    their KV heads together, matching gate and up rows together), the KV cache by KV head, and each
    sharded output that a later kernel reads whole is all-gathered (`gather` callback).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass

import numpy as np

from . import kernels as K


@dataclass
class DenseConfig:
    layers: int = 32
    hidden: int = 4096
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ff: int = 14336
    vocab: int = 128256
    rope_base: float = 500000.0
    eps: float = 1e-5
    max_ctx: int = 8192 + 64
    body_type: str = "q4_k"
    head_type: str = "q8_0"
    embed_type: str = "q4_k"

    @property
    def q_dim(self):
        return self.heads * self.head_dim

    @property
    def kv_dim(self):
        return self.kv_heads * self.head_dim


def shard_rows(total: int, rank: int, world: int):
    """Rows [lo, hi) of `total` that rank owns (contiguous, equal parts)."""
    assert total % world == 0, (total, world)
    per = total // world
    return rank * per, (rank + 1) * per


@dataclass
class Shard:
    """What one rank holds of the model (world = 1: everything)."""
    rank: int = 0
    world: int = 1

    def heads(self, cfg: DenseConfig):
        return shard_rows(cfg.heads, self.rank, self.world)

    def kv_heads(self, cfg: DenseConfig):
        return shard_rows(cfg.kv_heads, self.rank, self.world)


def layer_weight_shapes(cfg: DenseConfig, sh: Shard):
    """name -> (rows held by this rank, k) for every matrix of a layer."""
    h0, h1 = sh.heads(cfg)
    g0, g1 = sh.kv_heads(cfg)
    hd = cfg.head_dim
    ff0, ff1 = shard_rows(cfg.ff, sh.rank, sh.world)
    e0, e1 = shard_rows(cfg.hidden, sh.rank, sh.world)
    return {
        "wqkv": ((h1 - h0) * hd + 2 * (g1 - g0) * hd, cfg.hidden),
        "wo": (e1 - e0, cfg.q_dim),
        "wgu": (2 * (ff1 - ff0), cfg.hidden),
        "wdown": (e1 - e0, cfg.ff),
    }


def slice_full_weights(cfg: DenseConfig, sh: Shard, name: str, full: np.ndarray) -> np.ndarray:
    """The rows of a full (unsharded, stacked) weight matrix [rows, row_bytes] that this rank holds, in
    the order the sharded program expects. Used by tests to shard one seeded model for every world size."""
    hd = cfg.head_dim
    h0, h1 = sh.heads(cfg)
    g0, g1 = sh.kv_heads(cfg)
    if name == "wqkv":
        q = full[h0 * hd:h1 * hd]
        k = full[cfg.q_dim + g0 * hd:cfg.q_dim + g1 * hd]
        v = full[cfg.q_dim + cfg.kv_dim + g0 * hd:cfg.q_dim + cfg.kv_dim + g1 * hd]
        return np.concatenate([q, k, v])
    if name == "wgu":
        f0, f1 = shard_rows(cfg.ff, sh.rank, sh.world)
        return np.concatenate([full[f0:f1], full[cfg.ff + f0:cfg.ff + f1]])
    if name in ("wo", "wdown"):
        e0, e1 = shard_rows(cfg.hidden, sh.rank, sh.world)
        return full[e0:e1]
    if name == "head":
        v0, v1 = shard_rows(cfg.vocab, sh.rank, sh.world)
        return full[v0:v1]
    raise KeyError(name)


class DenseProgram:
    """Buffers and the launch list of one decode step for `batch` sequences on one rank.

    `weights`: {"embed": buf, "head": buf, "out_norm": buf, "layers": [{"wqkv","wo","wgu","wdown",
    "attn_norm","ffn_norm"}]} of device buffers (anything with .ptr/.nbytes or (ptr, size)) in the kernels'
    layouts. `alloc(nbytes)` returns a zeroed device buffer. `gather(buf, batch, width_total)`, for
    world > 1, makes every rank's column slice of a [batch, width_total] f32 buffer visible on all ranks.
    """

    def __init__(self, ctx, cfg: DenseConfig, weights, batch: int, alloc, shard: Shard | None = None, gather=None,
                 variants: dict | None = None, fuse_rope: bool | None = None, arena=None, batched: bool | None = None):
        self.ctx, self.cfg, self.w, self.B = ctx, cfg, weights, batch
        self.sh = shard or Shard()
        self.gather = gather
        # Tensor parallelism without a collective library: `arena` (abi.PeerArena) holds the vectors every rank
        # reads whole; their producers store into every rank's arena and publish an exchange slot, their
        # consumers wait for it. Slots: 4 per layer (att, x after wo, act, x after down), then the logits.
        self.arena = arena
        assert arena is None or gather is None
        self.L = K.Launcher(ctx)
        self.variants = variants or {}
        # rope_append inside the Q|K|V multiply's epilogue (one launch fewer per layer) where that is built:
        # 1, 2 or 4 sequences
        self.fuse_rope = (batch in (1, 2, 4)) if fuse_rope is None else fuse_rope
        # Q4_K multiplies of 5..64 sequences in ONE pass over the weights (the tcgen05 family) instead of a pass per
        # 2-4 sequences
        can_batch = 4 < batch <= K.MATVEC_BATCHED_MAX_TOKENS
        self.batched = can_batch if batched is None else (bool(batched) and batch <= K.MATVEC_BATCHED_MAX_TOKENS)
        # attn_combine inside the output projection (one launch fewer per attention layer) where the projection takes
        # its input from an exchange and runs the tensor-core family of up to four sequences
        self.fuse_combine = arena is not None and not self.batched and batch <= 4 and cfg.body_type in ("q4_k", "q8_0")
        self.launches_per_step = 0
        sh, hd = self.sh, cfg.head_dim
        h0, h1 = sh.heads(cfg)
        g0, g1 = sh.kv_heads(cfg)
        self.lh, self.lg = h1 - h0, g1 - g0                  # local query / KV heads
        self.h0, self.g0 = h0, g0
        self.qkv_row = (self.lh + 2 * self.lg) * hd
        self.lff = cfg.ff // sh.world
        self.le = cfg.hidden // sh.world
        self.lv = cfg.vocab // sh.world
        B, e = batch, cfg.hidden
        f4 = 4
        self.tokens = alloc(B * 4)
        self.positions = alloc(B * 4)
        self.step = alloc(16)
        shared = arena.alloc if arena is not None else alloc
        self.x = shared(B * e * f4)
        self.qkv = alloc(B * self.qkv_row * f4)
        self.att = shared(B * cfg.q_dim * f4)         # full width: column slices are gathered
        self.act = shared(B * cfg.ff * f4)
        self.logits = shared(B * cfg.vocab * f4)
        self.max_blocks = -(-cfg.max_ctx // K.ATTN_BLOCK)
        self.part = alloc(B * self.lh * self.max_blocks * (hd + 2) * f4)
        self.seq_stride = cfg.max_ctx * self.lg * hd          # cache elements per sequence
        self.kc = [alloc(B * self.seq_stride * 2) if self._has_cache(il) else None for il in range(cfg.layers)]
        self.vc = [alloc(B * self.seq_stride * 2) if self._has_cache(il) else None for il in range(cfg.layers)]
        self.dummy = alloc(256)
        self.rope = None

    def _has_cache(self, il: int) -> bool:
        return True

    # ---- host-built tables and per-step state
    def set_rope_table(self, table_buf):
        """(cos, sin) per (position, pair), built on the host (src/kernels/kernels.zig:730-744)."""
        self.rope = table_buf

    @staticmethod
    def rope_table(cfg: DenseConfig) -> np.ndarray:
        """The table for every position of the context (normal RoPE, no per-pair factors)."""
        from . import abi

        return abi.rope_table(cfg.max_ctx, cfg.head_dim, cfg.rope_base)

    def write_step(self, tokens: np.ndarray, positions: np.ndarray):
        """The step's inputs: one token id and one position per sequence."""
        assert tokens.size == self.B and positions.size == self.B
        self.tokens.upload(np.ascontiguousarray(tokens, dtype=np.uint32))
        self.positions.upload(np.ascontiguousarray(positions, dtype=np.uint32))
        self.step.upload(np.array([self.B, int(positions[0]), 0, 0], dtype=np.uint32))

    # ---- the launch list
    def _matvec(self, ttype, x, w, out, n, k, **kw):
        v = self.variants.get((ttype, n, k), 0)
        if v == 0 and self.batched and ttype == "q4_k" and k % 256 == 0 and "rope" not in kw:
            v = K.MATVEC_BATCHED
        self.L.matvec(ttype, x, w, out, n, k, m=self.B, variant=v, **kw)
        self.launches_per_step += 3 if v == K.MATVEC_BATCHED else 1  # columns, multiply, reduction

    def _runs_16_warp_mma(self, ttype, n, k) -> bool:
        """Whether the shape's multiply runs the tensor-core family in CTAs of 16 warps (the form that can take
        attn_combine as its first phase)."""
        v = self.variants.get((ttype, n, k), 0)
        if v == 0:
            return k % 256 == 0
        return (v >> 16) & 0xFF == K.FAMILY_MMA and (v >> 8) & 0x0F == K.SHAPE_16_WARPS

    def sweep(self, tokens: int | None = None) -> dict:
        """The load-time sweep over this program's multiply shapes on the model's own weights (tune.Sweep, the
        counterpart of src/tune/tune.zig; every layer's matrix of a shape takes its turn, so the timings are of
        weights that come from HBM). Takes the table for the launches recorded from now on and returns it."""
        from . import tune

        s = tune.Sweep(self.ctx, tokens=min(tokens or self.B, 4))
        self._sweep_shapes(s)
        table = s.run()
        self.variants = {**self.variants, **table}
        self.sweep_report = s.report
        return table

    @staticmethod
    def pick_trial(times, margin: float, agree=None) -> int:
        """Which of a shape's trials stays (times[0] is the default form's step): the fastest, if it beats the default
        by more than `margin`, else the default. `agree` maps this rank's times to the ones every rank decides by
        (the maximum over ranks: a step ends when its slowest rank does), so that all ranks keep the SAME trial - a
        combination of forms that was timed, not one per rank from different trials."""
        times = list(times) if agree is None else list(agree(list(times)))
        best = min(range(len(times)), key=lambda i: times[i])
        return best if times[best] < times[0] * (1.0 - margin) else 0

    def refine(self, max_keys: int, top: int = 3, reps: int = 10, margin: float = 0.005, agree=None) -> dict:
        """After sweep(): every shape goes back to the library's default form; then, shape by shape (largest first),
        the default and the `top` candidates that were fastest on their own are tried inside the replayed step, and a
        candidate replaces the default only where it makes the STEP faster by more than `margin`. A multiply's time
        in the step depends on its neighbours (what the kernel before it leaves in flight, how its ring depth meets
        the next kernel's start): the form that wins alone is often not the one that wins there, and the best few
        lie within the sweep's noise of each other, so the stand-alone figures only nominate. Starting from the
        defaults makes the result no slower than an untuned program (up to the margin). Every rank of a
        tensor-parallel program runs the same number of steps here (`top` + 1 trials per shape), as the exchange
        requires, and with `agree` (see pick_trial) they all keep the same trial of a shape."""
        import time

        by_shape = {}
        for ttype, n, k, variant, ns in getattr(self, "sweep_report", []):
            if ns is not None:
                by_shape.setdefault((ttype, n, k), []).append((ns, variant))

        def step_seconds() -> float:
            self.ctx.capture_begin()
            self.record_step(max_keys)
            g = self.ctx.capture_end()
            for _ in range(2):
                self.ctx.graph_launch(g)
            self.ctx.sync()
            best = float("inf")
            for _ in range(3):
                t0 = time.perf_counter()
                for _ in range(reps):
                    self.ctx.graph_launch(g)
                self.ctx.sync()
                best = min(best, (time.perf_counter() - t0) / reps)
            self.ctx.graph_destroy(g)
            return best

        for shape in by_shape:
            self.variants[shape] = 0
        self.refine_report = []
        for shape in sorted(by_shape, key=lambda s: -s[1] * s[2]):
            trials = [v for _, v in sorted(by_shape[shape]) if v != 0 and v != K.MATVEC_DEFAULT_FORM.get(shape[0])][:top]
            trials = [0] + trials + [0] * (top - len(trials))
            timed = []
            for v in trials:
                self.variants[shape] = v
                timed.append((step_seconds(), v))
            self.variants[shape] = trials[self.pick_trial([t for t, _ in timed], margin, agree)]
            self.refine_report.append((shape, timed))
        return self.variants

    def _sweep_shapes(self, s):
        cfg, e = self.cfg, self.cfg.hidden
        layers = self.w["layers"]
        att = [lw for lw in layers if "wqkv" in lw]
        s.add(cfg.body_type, [lw["wqkv"] for lw in att], self.qkv_row, e, flags=K.NORM, eps=cfg.eps, norm_w=att[0]["attn_norm"])
        s.add(cfg.body_type, [lw["wo"] for lw in att], self.le, cfg.q_dim)
        s.add(cfg.body_type, [lw["wgu"] for lw in layers], self.lff, e, flags=K.NORM | K.SILU_PAIR, eps=cfg.eps, half=self.lff,
              norm_w=layers[0]["ffn_norm"])
        s.add(cfg.body_type, [lw["wdown"] for lw in layers], self.le, cfg.ff)
        s.add(cfg.head_type, self.w["head"], self.lv, e, flags=K.NORM, eps=cfg.eps, norm_w=self.w["out_norm"])

    def _gather(self, buf, width):
        if self.gather is not None:
            self.gather(buf, self.B, width)

    @staticmethod
    def arena_bytes(cfg: DenseConfig, batch: int) -> int:
        """Bytes of the vectors a peer arena must hold for `batch` sequences (each rounded up to 256)."""
        return sum(((batch * w * 4 + 255) & ~255) for w in (cfg.hidden, cfg.q_dim, cfg.ff, cfg.vocab))

    @staticmethod
    def arena_slots(cfg: DenseConfig) -> int:
        return 4 * cfg.layers + 1

    def record_step(self, max_keys: int):
        """Issues the step's launches on the context's stream (inside a graph capture they are captured).
        `max_keys`: the largest position + 1 of the batch (sizes the attention grid)."""
        cfg, B, e = self.cfg, self.B, self.cfg.hidden
        self.launches_per_step = 0
        self._max_keys = max_keys
        # embedding rows of the step's tokens (replicated on every rank)
        self.L.embed(cfg.embed_type, self.tokens, self.w["embed"], self.x, B, e, 0, cfg.vocab)
        self.launches_per_step += 1
        for il in range(cfg.layers):
            self._mixer(il)
            self._ffn(il)
        self._head()

    def _slots(self, il):
        """The layer's four exchanges (mixer output, x after the mixer's output projection, the FFN activations, x
        after down) and the one its input x arrived under."""
        if self.arena is None:
            return (None,) * 5
        return 4 * il, 4 * il + 1, 4 * il + 2, 4 * il + 3, ((4 * il - 1) if il > 0 else None)

    def _mixer(self, il):
        """Attention: the reference's LayerBuilder.attention (src/plan/qwen35.zig:989-1036)."""
        cfg, B, hd, sh, e = self.cfg, self.B, self.cfg.head_dim, self.sh, self.cfg.hidden
        lw = self.w["layers"][il]
        s_att, s_xwo, _, _, s_prev = self._slots(il)
        rp = K.RopeAppend(self.lh, self.lg, hd, hd, self.qkv_row, self.lh * hd, (self.lh + self.lg) * hd, K.KV_F16,
                          cfg.eps, 0, 0, 1, 0)
        rp._pad[0] = self.seq_stride
        ap = K.Attention(self.lh, self.lg, hd, K.KV_F16, K.attention_scale(hd), self.max_blocks, self.qkv_row, 0, 0, 0)
        ap._pad[0] = self.seq_stride
        ap._pad[1] = cfg.q_dim                                  # att rows are full width on every rank
        blocks = -(-self._max_keys // K.ATTN_BLOCK)
        att_cols = self.att.at(self.h0 * hd * 4)                # this rank's head columns of att
        # 1. fused attn_norm + Q|K|V projection (local heads); 2. RoPE (normal pairs) and the cache append at
        #    each sequence's position, in the multiply's epilogue or as rope_append's own launch
        if self.fuse_rope:
            self._matvec(cfg.body_type, self.x, lw["wqkv"], self.qkv, self.qkv_row, e, flags=K.NORM, eps=cfg.eps,
                         norm_w=lw["attn_norm"], rope=(rp, [self.rope, self.kc[il], self.vc[il], self.step, self.positions]),
                         wait=s_prev)
        else:
            self._matvec(cfg.body_type, self.x, lw["wqkv"], self.qkv, self.qkv_row, e, flags=K.NORM, eps=cfg.eps,
                         norm_w=lw["attn_norm"], wait=s_prev)
            self.L.launch(K.ROPE_APPEND, rp, [self.qkv, self.dummy, self.dummy, self.rope, self.kc[il], self.vc[il],
                                              self.step, self.positions], (self.lh + self.lg, B, 1))
            self.launches_per_step += 1
        # 3-4. split attention over each sequence's cache, merged into this rank's head columns of att
        self.L.launch(K.ATTN_SPLIT, ap, [self.qkv, self.kc[il], self.vc[il], self.part, self.step, self.positions],
                      (self.lg, blocks, B), self.variants.get("attn_split", 0))
        fused = self.fuse_combine and self._runs_16_warp_mma(cfg.body_type, self.le, cfg.q_dim)
        if not fused:
            self.L.launch(K.ATTN_COMBINE, K.with_peer(ap, push=s_att), [self.qkv, self.part, att_cols, self.step, self.positions],
                          (self.lh, B, 1))
        self.launches_per_step += 1 if fused else 2
        self._gather(self.att, cfg.q_dim)
        # 5. Wo rows of this rank, accumulated into the residual stream's slice (with the merge of the attention's
        #    partials as its first phase, when fused)
        self._matvec(cfg.body_type, self.att, lw["wo"], self.x, self.le, cfg.q_dim, col0=sh.rank * self.le,
                     out_stride=e, flags=K.ACCUMULATE, wait=s_att, push=s_xwo,
                     **({"combine": (ap, [self.qkv, self.part, att_cols, self.step, self.positions])} if fused else {}))
        self._gather(self.x, e)

    def _ffn(self, il):
        """LayerBuilder.ffn (src/plan/qwen35.zig:1039-1052)."""
        cfg, sh, e = self.cfg, self.sh, self.cfg.hidden
        lw = self.w["layers"][il]
        _, s_xwo, s_act, s_xdown, _ = self._slots(il)
        # 6. fused ffn_norm + gate|up + SwiGLU (local ff rows)
        self._matvec(cfg.body_type, self.x, lw["wgu"], self.act, self.lff, e, col0=sh.rank * self.lff,
                     out_stride=cfg.ff, flags=K.NORM | K.SILU_PAIR, eps=cfg.eps, half=self.lff,
                     norm_w=lw["ffn_norm"], wait=s_xwo, push=s_act)
        self._gather(self.act, cfg.ff)
        # 7. Wdown rows of this rank, accumulated
        self._matvec(cfg.body_type, self.act, lw["wdown"], self.x, self.le, cfg.ff, col0=sh.rank * self.le,
                     out_stride=e, flags=K.ACCUMULATE, wait=s_act, push=s_xdown)
        self._gather(self.x, e)

    def _head(self):
        """The output norm fused into the LM head (src/plan/qwen35.zig:609)."""
        cfg, sh, e = self.cfg, self.sh, self.cfg.hidden
        peer = self.arena is not None
        s_logits = 4 * cfg.layers if peer else None
        self._matvec(cfg.head_type, self.x, self.w["head"], self.logits, self.lv, e, col0=sh.rank * self.lv,
                     out_stride=cfg.vocab, flags=K.NORM, eps=cfg.eps, norm_w=self.w["out_norm"],
                     wait=(4 * cfg.layers - 1) if peer else None, push=s_logits)
        self._gather(self.logits, cfg.vocab)
        if peer:
            self.L.peer_wait(s_logits, self.logits)  # the host may read the logits once this has run
            self.L.peer_next()                       # the next run of the list tags its exchanges anew
            self.launches_per_step += 2

    def algorithmic_bytes(self, positions: np.ndarray) -> dict:
        """Bytes one step must move on this rank: every weight once, K and V of every cached position."""
        cfg = self.cfg
        shapes = layer_weight_shapes(cfg, self.sh)
        body = sum(r * K.row_bytes(cfg.body_type, k) for r, k in shapes.values()) * cfg.layers
        head = self.lv * K.row_bytes(cfg.head_type, cfg.hidden)
        kv = sum(2 * (int(p) + 1) * self.lg * cfg.head_dim * 2 for p in positions) * cfg.layers
        return {"weights": body + head, "kv": kv, "total": body + head + kv}


@dataclass
class HybridConfig(DenseConfig):
    """A Qwen 3.5-style hybrid: Gated DeltaNet layers with a full-attention layer every `attention_every` layers
    (src/graph/qwen35.zig:21-56). DeltaNet: `gdn_v_heads` value heads over `gdn_k_heads` key heads (value head j
    uses key head j mod k_heads) of `gdn_head_dim`, a causal depthwise conv of `conv_kernel` taps."""
    gdn_head_dim: int = 128
    gdn_k_heads: int = 16
    gdn_v_heads: int = 16
    conv_kernel: int = 4
    attention_every: int = 4

    def is_attention(self, il: int) -> bool:
        return (il + 1) % self.attention_every == 0

    @property
    def gdn_inner(self):
        return self.gdn_v_heads * self.gdn_head_dim


def delta_shard(cfg: HybridConfig, sh: Shard):
    """(first value head, value heads, first key head, key heads) a rank holds: value heads are cut into contiguous
    equal parts; a rank keeps the key heads its value heads use (j mod k_heads: a contiguous run)."""
    v0, v1 = shard_rows(cfg.gdn_v_heads, sh.rank, sh.world)
    lv = v1 - v0
    lk = min(lv, cfg.gdn_k_heads)
    k0 = v0 % cfg.gdn_k_heads
    assert lv % lk == 0 and k0 + lk <= cfg.gdn_k_heads and cfg.gdn_v_heads % cfg.gdn_k_heads == 0, (v0, lv, k0, lk)
    return v0, lv, k0, lk


def slice_delta_weights(cfg: HybridConfig, sh: Shard, name: str, full: np.ndarray) -> np.ndarray:
    """A rank's rows of a DeltaNet layer's full matrices / vectors (model.hybrid_host_model's names)."""
    d, hk, hv = cfg.gdn_head_dim, cfg.gdn_k_heads, cfg.gdn_v_heads
    v0, lv, k0, lk = delta_shard(cfg, sh)
    key, inner = hk * d, hv * d
    if name in ("wproj", "conv"):
        # rows (channels): q heads | k heads | v heads [| z heads | beta | alpha]
        parts = [full[k0 * d:(k0 + lk) * d], full[key + k0 * d:key + (k0 + lk) * d], full[2 * key + v0 * d:2 * key + (v0 + lv) * d]]
        if name == "wproj":
            z0 = 2 * key + inner
            parts += [full[z0 + v0 * d:z0 + (v0 + lv) * d], full[z0 + inner + v0:z0 + inner + v0 + lv],
                      full[z0 + inner + hv + v0:z0 + inner + hv + v0 + lv]]
        return np.concatenate(parts)
    if name in ("dt_bias", "a"):
        return full[v0:v0 + lv]
    if name == "wout":
        e0, e1 = shard_rows(cfg.hidden, sh.rank, sh.world)
        return full[e0:e1]
    raise KeyError(name)


class HybridProgram(DenseProgram):
    """The decode step of a hybrid model for ONE sequence (the DeltaNet kernels take a step's rows as consecutive
    tokens of one sequence, as the reference does): attention layers as in DenseProgram, DeltaNet layers as the
    reference's plan builds them (src/plan/qwen35.zig:556-599):
        proj = matvec(x, wproj, NORM)   rows q | k | v | z | beta | alpha of the rank's heads
        delta_prep -> delta_rule -> gated_norm     (conv history and state per layer; o = the rank's head columns)
        x += matvec(o, wout)            the output projection reads o whole: one exchange, like attention's
    then the FFN. With W ranks the value heads are sharded (delta_shard), so is every state.
    A DeltaNet layer's weights: {"wproj", "conv", "dt_bias", "a", "norm", "wout", "attn_norm", "ffn_norm", "wgu", "wdown"}."""

    def __init__(self, ctx, cfg: HybridConfig, weights, batch: int, alloc, shard: Shard | None = None, **kw):
        assert batch == 1, "a hybrid step is one sequence"
        super().__init__(ctx, cfg, weights, batch, alloc, shard, **kw)
        d, taps = cfg.gdn_head_dim, cfg.conv_kernel
        self.v0, self.lvh, self.k0, self.lkh = delta_shard(cfg, self.sh)
        self.conv_dim = 2 * self.lkh * d + self.lvh * d
        self.proj_row = self.conv_dim + self.lvh * d + 2 * self.lvh
        shared = self.arena.alloc if self.arena is not None else alloc
        self.proj = alloc(self.proj_row * 4)
        self.conv = alloc(self.conv_dim * 4)
        self.g, self.beta = alloc(max(256, self.lvh * 4)), alloc(max(256, self.lvh * 4))
        self.o = shared(cfg.gdn_inner * 4)                                # full width: head columns are exchanged
        self.state = {il: alloc(self.lvh * d * d * 4) for il in range(cfg.layers) if not cfg.is_attention(il)}
        self.hist = {il: alloc((taps - 1) * self.conv_dim * 4) for il in range(cfg.layers) if not cfg.is_attention(il)}

    def _has_cache(self, il: int) -> bool:
        return self.cfg.is_attention(il)

    def _sweep_shapes(self, s):
        super()._sweep_shapes(s)
        cfg = self.cfg
        delta = [lw for lw in self.w["layers"] if "wproj" in lw]
        s.add(cfg.body_type, [lw["wproj"] for lw in delta], self.proj_row, cfg.hidden, flags=K.NORM, eps=cfg.eps, norm_w=delta[0]["attn_norm"])
        s.add(cfg.body_type, [lw["wout"] for lw in delta], self.le, cfg.gdn_inner)

    @staticmethod
    def arena_bytes(cfg, batch: int) -> int:
        return DenseProgram.arena_bytes(cfg, batch) + ((batch * cfg.gdn_inner * 4 + 255) & ~255)

    def _mixer(self, il):
        cfg = self.cfg
        if cfg.is_attention(il):
            return super()._mixer(il)
        sh, e, d = self.sh, cfg.hidden, cfg.gdn_head_dim
        lw = self.w["layers"][il]
        s_o, s_xwo, _, _, s_prev = self._slots(il)
        self._matvec(cfg.body_type, self.x, lw["wproj"], self.proj, self.proj_row, e, flags=K.NORM, eps=cfg.eps,
                     norm_w=lw["attn_norm"], wait=s_prev)
        inner = self.lvh * d
        pp = K.DeltaPrep(self.conv_dim, cfg.conv_kernel, 2 * self.lkh * d, d, self.proj_row, self.lvh, self.conv_dim + inner,
                         self.conv_dim + inner + self.lvh, cfg.eps)
        self.L.delta_prep(pp, self.proj, lw["conv"], self.hist[il], self.conv, lw["dt_bias"], lw["a"], self.g, self.beta, 1)
        o_cols = self.o.at(self.v0 * d * 4)                               # this rank's head columns of o
        pr = K.DeltaRule(self.lkh, self.lvh, d, self.conv_dim, cfg.conv_kernel, self.proj_row, 0)
        self.L.delta_rule(pr, self.conv, self.g, self.beta, self.state[il], o_cols, self.step, self.proj, self.hist[il], self.dummy)
        gn = K.GatedNorm(self.lvh, d, cfg.eps, self.proj_row, self.conv_dim, 0)
        self.L.launch(K.GATED_NORM, K.with_peer(gn, push=s_o), [o_cols, self.proj, lw["norm"]], (self.lvh, 1, 1))
        self.launches_per_step += 3
        self._gather(self.o, cfg.gdn_inner)
        self._matvec(cfg.body_type, self.o, lw["wout"], self.x, self.le, cfg.gdn_inner, col0=sh.rank * self.le, out_stride=e,
                     flags=K.ACCUMULATE, wait=s_o, push=s_xwo)
        self._gather(self.x, e)

