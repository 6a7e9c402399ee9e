"""Kernel identities, parameter blocks and launch helpers: the host-side mirror
of the reference's kernel catalog (src/kernels/kernels.zig) for the CUDA backend.

Identities are `@intFromEnum(Kernel)` (kernels.zig:24-101); parameter blocks are
its `params.*` extern structs (kernels.zig:432-650); `Launcher.launch` takes the
same (kernel, params, args, groups) as the reference's (kernels.zig:938-960).
"""
from __future__ import annotations

import ctypes as C
import math

from . import abi

# kernels.Kernel
RMSNORM, MATMUL_BF16, MATMUL_F16, MATMUL_REDUCE, MATVEC_BF16, MATVEC_F16, SILU_MUL = 0, 1, 2, 3, 4, 5, 6
EMBED_BF16, EMBED_F16, ROPE_APPEND, ATTN_SPLIT, ATTN_SPLIT_WIDE, ATTN_SPLIT_SPARSE, ATTN_COMBINE = 7, 8, 9, 10, 11, 12, 13
DELTA_PREP, DELTA_RULE, GATED_NORM = 18, 19, 20
MARK_TOKENS, SAMPLE, DRAFT = 21, 22, 23
REPAD, REPACK_Q3_K = 36, 37
REPACK_Q8_0, QUANTIZE_Q8, MATVEC_Q8_0, MATVEC_Q4_K = 38, 39, 40, 42
MATVEC_Q3_K, MATVEC_Q5_K, MATVEC_Q6_K = 41, 43, 44
EMBED_Q3_K, EMBED_Q5_K, EMBED_Q6_K, EMBED_IQ4_XS = 52, 54, 55, 56
MATMUL_Q8_0, MATMUL_Q4_K, EMBED_Q8_0, EMBED_Q4_K = 45, 48, 51, 53
MATMUL_Q8_0_FLOAT = 46
KERNEL_COUNT = 57

# MatvecBf16.Flags (kernels.zig:485-493)
NORM, ACCUMULATE, SILU_PAIR = 1, 2, 4
# an extension of this backend: the multiply's outputs are a Q|K|V row, rotated and appended to the cache in its
# epilogue (rope_append without its own launch); the parameter block is Matvec followed by RopeAppend
ROPE_APPEND_FUSED = 8
# likewise: the multiply reads the attention output and merges the attention's partials into it first (attn_combine
# without its own launch); the parameter block is Matvec followed by Attention, the multiply waits on an exchange
ATTN_COMBINE_FUSED = 16

# plan.common.KvFormat
KV_F32, KV_F16, KV_FP8 = 0, 1, 2

ATTN_BLOCK = 64        # kernels.attn_block
ATTN_ROWS = 32         # kernels.attn_rows
DECODE_MAX_ROWS = 4    # kernels.decode_max_rows
ATTN_MAX_GROUP = 8     # kernels.attn_max_group
ATTN_MAX_GROUP_WIDE = 12

FAMILY_SCALAR, FAMILY_MMA, FAMILY_TCGEN05 = 1, 2, 3


def variant(tiles: int = 0, splitk: int = 0, family: int = 0) -> int:
    """ZCU_VARIANT: this backend's matvec variant word (0 = default)."""
    return tiles | (splitk << 8) | (family << 16)


# Candidates the tuning sweep tries (the cuda arm of MatvecVariant.candidates, src/kernels/kernels.zig:365-373: there
# workgroup size x lanes per row x rows per lane; here the knobs this backend's multiply has). Tensor-core family:
# tiles in flight per warp (byte 0: 3..6), CTA shape (byte 1, low nibble: 0 = 16 warps and one CTA per SM, 1 = 8
# warps and two), CTA count (byte 1, bit 4: 0 = the count that divides the row tiles evenly, 1 = a CTA on every SM);
# scalar family: one shape.
SHAPE_16_WARPS, SHAPE_8_WARPS, GRID_EVERY_SM = 0, 1, 0x10
# what variant word 0 resolves to in the library, where a candidate names the same form (such a candidate is a repeat)
MATVEC_DEFAULT_FORM = {"q4_k": variant(3, SHAPE_16_WARPS | GRID_EVERY_SM, FAMILY_MMA)}
MATVEC_CANDIDATES = ([variant(st, shape | grid, FAMILY_MMA) for st in (3, 4, 5, 6) for shape in (SHAPE_16_WARPS, SHAPE_8_WARPS)
                      for grid in (0, GRID_EVERY_SM)] + [variant(0, 0, FAMILY_SCALAR)])
# matvec_q4_k for up to 64 tokens in one pass over the weights (tcgen05, accumulators in tensor memory).
MATVEC_BATCHED = variant(0, 0, FAMILY_TCGEN05)
MATVEC_BATCHED_MAX_TOKENS = 64


def matvec_variant_exists(ttype: str, k: int, v: int) -> bool:
    """Whether variant word `v` can run a (ttype, k) multiply: the tensor-core family needs Q8_0 rows of whole
    256-weight pieces (the default falls back to the scalar family there)."""
    family = (v >> 16) & 0xFF
    if family == FAMILY_TCGEN05:
        return ttype == "q4_k" and k % 256 == 0 and (v & 0xFFFF) == 0
    if ttype == "q8_0" and k % 256 != 0:
        return v == 0 or family == FAMILY_SCALAR
    return True

u32, f32 = C.c_uint32, C.c_float


def _struct(name, fields):
    return type(name, (C.Structure,), {"_fields_": fields})


Step = _struct("Step", [("m", u32), ("pos0", u32), ("u", f32), ("keep", u32)])
RmsNorm = _struct("RmsNorm", [("rows", u32), ("dim", u32), ("eps", f32), ("w_rows", u32)])
MatmulBf16 = _struct("MatmulBf16", [("rows", u32), ("n", u32), ("k", u32), ("col0", u32), ("out_stride", u32),
                                    ("accumulate", u32), ("_pad", u32 * 2)])
Matvec = _struct("MatvecBf16", [("n", u32), ("k", u32), ("col0", u32), ("out_stride", u32), ("eps", f32),
                                ("flags", u32), ("half", u32), ("x_stride", u32)])
RepackQ80 = _struct("RepackQ80", [("rows", u32), ("k", u32), ("_pad", u32 * 2)])
SiluMul = _struct("SiluMul", [("count", u32), ("width", u32), ("_pad", u32 * 2)])
Embed = _struct("EmbedBf16", [("dim", u32), ("row0", u32), ("chunk_rows", u32), ("stride", u32)])
RopeAppend = _struct("RopeAppend", [("heads", u32), ("kv_heads", u32), ("head_dim", u32), ("n_rot", u32), ("row", u32),
                                    ("k_off", u32), ("v_off", u32), ("kv", u32), ("eps", f32), ("gated", u32),
                                    ("qk_norm", u32), ("normal", u32), ("scales", u32), ("_pad", u32 * 3)])
QuantizeQ8 = _struct("QuantizeQ8", [("k", u32), ("block", u32), ("mode", u32), ("eps", f32)])
MatmulQuant = _struct("MatmulQuant", [("rows", u32), ("n", u32), ("k", u32), ("col0", u32), ("out_stride", u32),
                                      ("accumulate", u32), ("k_slice", u32), ("slice_stride", u32)])
MatmulReduce = _struct("MatmulReduce", [("rows", u32), ("n", u32), ("slices", u32), ("col0", u32), ("out_stride", u32),
                                        ("accumulate", u32), ("slice_stride", u32), ("_pad", u32)])
MatvecRope = _struct("MatvecRope", [("mv", Matvec), ("rope", RopeAppend)])
Attention = _struct("Attention", [("heads", u32), ("kv_heads", u32), ("head_dim", u32), ("kv", u32), ("scale", f32),
                                  ("max_blocks", u32), ("q_row", u32), ("row0", u32), ("gated", u32), ("scales", u32),
                                  ("_pad", u32 * 2)])
MatvecCombine = _struct("MatvecCombine", [("mv", Matvec), ("attn", Attention)])
DeltaPrep = _struct("DeltaPrep", [("channels", u32), ("taps", u32), ("key_channels", u32), ("head", u32), ("row", u32),
                                  ("v_heads", u32), ("beta_off", u32), ("alpha_off", u32), ("eps", f32),
                                  ("_pad", u32 * 3)])
DeltaRule = _struct("DeltaRule", [("k_heads", u32), ("v_heads", u32), ("dim", u32), ("conv_stride", u32), ("taps", u32),
                                  ("row", u32), ("kept_hist", u32), ("_pad", u32)])
GatedNorm = _struct("GatedNorm", [("v_heads", u32), ("dim", u32), ("eps", f32), ("z_row", u32), ("z_off", u32),
                                  ("sigmoid", u32), ("_pad", u32 * 2)])

assert C.sizeof(Matvec) == 32 and C.sizeof(RopeAppend) == 64 and C.sizeof(Attention) == 48
assert C.sizeof(DeltaPrep) == 48 and C.sizeof(DeltaRule) == 32 and C.sizeof(GatedNorm) == 32

# The sampler (kernels.zig:424-430, 622-725)
MAX_BIAS, MAX_STOPS, SAMPLE_SPAN, SAMPLE_CAP, SAMPLE_BISECT_ROUNDS = 1024, 16, 1024, 1024, 32
Sample = _struct("Sample", [("vocab", u32), ("n_bias", u32), ("n_stop", u32), ("greedy", u32), ("temperature", f32),
                            ("top_k", u32), ("top_p", f32), ("min_p", f32), ("repetition", f32), ("presence", f32),
                            ("frequency", f32), ("n_prompt", u32), ("stops", u32 * MAX_STOPS)])
SamplePhase = _struct("SamplePhase", [("phase", u32), ("round", u32), ("_pad", u32 * 2)])
Draft = _struct("Draft", [("vocab", u32), ("row", u32), ("slot", u32), ("_pad", u32)])
assert C.sizeof(Sample) == 112 and C.sizeof(SamplePhase) == 16 and C.sizeof(Draft) == 16
(PH_PREP, PH_REDUCE, PH_HIST, PH_DIGIT, PH_GATHER, PH_FINAL, PH_MASS, PH_PICK, PH_BISECT_INIT, PH_BISECT_MASS,
 PH_BISECT_STEP, PH_UNBUMP) = range(12)
WIDE_PHASES = (PH_PREP, PH_HIST, PH_GATHER, PH_MASS, PH_BISECT_MASS)
GREEDY_BELOW = 1e-5   # sampler.greedy_below


def sample_params(vocab: int, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repetition=1.0, presence=0.0, frequency=0.0,
                  n_bias=0, stops=(), n_prompt=0) -> "Sample":
    """Params.gpu (src/sampler/sampler.zig:58-79)."""
    assert len(stops) <= MAX_STOPS and n_bias <= MAX_BIAS
    s = Sample(vocab, n_bias, len(stops), int(temperature < GREEDY_BELOW), temperature, 0 if top_k >= vocab else top_k, top_p, min_p,
               repetition, presence, frequency, n_prompt)
    for i, t in enumerate(stops):
        s.stops[i] = t
    return s


def sample_steps(s: "Sample"):
    """The (phase, round) dispatches of one draw: kernels.sampleSteps (kernels.zig:683-715). This backend makes the
    draw in the first of them and accepts the rest without launching."""
    steps = [(PH_PREP, 0), (PH_REDUCE, 0)]
    if s.greedy:
        return steps
    if s.top_k > 0:
        for r in range(4):
            steps += [(PH_HIST, r), (PH_DIGIT, r)]
    if s.top_p < 1 and s.top_k > 0 and s.top_k <= SAMPLE_CAP:
        return steps + [(PH_GATHER, 0), (PH_FINAL, 0)]
    if s.top_p < 1:
        steps += [(PH_MASS, 0), (PH_BISECT_INIT, 0)] + [(PH_BISECT_MASS, 0), (PH_BISECT_STEP, 0)] * SAMPLE_BISECT_ROUNDS
    return steps + [(PH_MASS, 0), (PH_PICK, 0)]


def sample_groups(vocab: int) -> int:
    return -(-vocab // SAMPLE_SPAN)


def sample_state_words(vocab: int) -> int:
    return 16 + 256 + 2 * sample_groups(vocab) + 2 * SAMPLE_CAP


# Bytes per 256-weight block as the kernels read it (kernels.blockStride, kernels.zig:137-151) and as the file holds it.
BLOCK_STRIDE = {"q3_k": 128, "q5_k": 176, "q6_k": 224, "iq4_xs": 144}
FILE_BLOCK = {"q3_k": 110, "q5_k": 176, "q6_k": 210, "iq4_xs": 136}
Repad = _struct("Repad", [("blocks", u32), ("src_bytes", u32), ("dst_bytes", u32), ("_pad", u32)])
RepackQ3K = _struct("RepackQ3K", [("blocks", u32), ("_pad", u32 * 3)])


def row_bytes(ttype: str, k: int) -> int:
    """Bytes per row as the kernels read it (kernels.rowBytes, kernels.zig:157-160)."""
    if ttype == "q8_0":
        return (k + k // 16 + 15) & ~15
    if ttype == "q4_k":
        return k // 256 * 144
    if ttype in BLOCK_STRIDE:
        return k // 256 * BLOCK_STRIDE[ttype]
    if ttype in ("bf16", "f16"):
        return 2 * k
    raise ValueError(ttype)


MATVEC_KERNEL = {"q4_k": MATVEC_Q4_K, "q8_0": MATVEC_Q8_0, "bf16": MATVEC_BF16, "f16": MATVEC_F16, "q3_k": MATVEC_Q3_K, "q5_k": MATVEC_Q5_K,
                 "q6_k": MATVEC_Q6_K}
EMBED_KERNEL = {"q4_k": EMBED_Q4_K, "q8_0": EMBED_Q8_0, "bf16": EMBED_BF16, "f16": EMBED_F16, "q3_k": EMBED_Q3_K, "q5_k": EMBED_Q5_K,
                "q6_k": EMBED_Q6_K, "iq4_xs": EMBED_IQ4_XS}


def elementwise(count: int):
    """Launcher.elementwise (kernels.zig:981-986)."""
    groups = -(-count // 256)
    if groups <= 65535:
        return (groups, 1, 1)
    return (65535, -(-groups // 65535), 1)


# The reserved variant of the lower-precision prefill rung (src/agility/kernels.zig:116-122) and the layout
# bits this backend reads from MatmulBf16._pad[0] under it.
VARIANT_PREFILL_TC = 0xFFFC0000
X_HALF, OUT_HALF = 1, 2
# delta_rule in 64-token chunks; DeltaRule._pad carries the step's token count.
VARIANT_DELTA_CHUNK64 = 0xFFFD0000
VARIANT_DELTA_CHUNK64_F32 = 0xFFFD0001   # the same form in f32 on the CUDA cores


# The tensor-parallel exchange a dispatch takes part in (zcu_peer_ext): appended to its parameter block.
PEER_MAGIC, PEER_NONE, EXT_PEER_WAIT, EXT_PEER_NEXT = 0x52454550, 0xFFFFFFFF, 64, 65
PeerExt = _struct("PeerExt", [("magic", u32), ("wait_slot", u32), ("push_slot", u32), ("reserved", u32)])


def with_peer(params, wait=None, push=None):
    """`params` followed by a PeerExt (or `params` itself when the dispatch takes no part in an exchange)."""
    if wait is None and push is None:
        return params
    ext = PeerExt(PEER_MAGIC, PEER_NONE if wait is None else wait, PEER_NONE if push is None else push, 0)
    raw = bytes(params) + bytes(ext)
    return (C.c_uint8 * len(raw)).from_buffer_copy(raw)


class Launcher:
    """Immediate launches on a context (kernels.Launcher, kernels.zig:925-960)."""

    def __init__(self, ctx: abi.Context):
        self.ctx = ctx

    def launch(self, kernel: int, params, args, groups, variant: int = 0):
        self.ctx.launch(kernel, params, args, groups, variant)

    # -- the decode multiply: grid (ceil(n / groupRows), m, 1) in the reference; only m matters here
    def matvec(self, ttype, x, w, out, n, k, m=1, col0=0, out_stride=None, flags=0, eps=0.0, half=0, x_stride=0,
               norm_w=None, variant=0, rope=None, wait=None, push=None, combine=None):
        """`rope` = (RopeAppend, [table, kc, vc, step(, positions)]) fuses rope_append into the multiply that
        produces the Q|K|V row (ROPE_APPEND_FUSED; needs norm_w as binding 3). `combine` = (Attention, [qg, part,
        out, step(, positions)]) fuses attn_combine into the multiply that reads the attention output
        (ATTN_COMBINE_FUSED; the multiply must `wait` on the exchange the merged heads are pushed under)."""
        p = Matvec(n, k, col0, out_stride if out_stride is not None else n, eps, flags, half, x_stride)
        args = [x, w, out] + ([norm_w] if norm_w is not None else [])
        if combine is not None:
            assert rope is None and wait is not None
            p.flags |= ATTN_COMBINE_FUSED
            p = MatvecCombine(p, combine[0])
            args = (args + [x])[:4] + list(combine[1])   # binding 3 (norm weights) is a placeholder when there is no norm
        if rope is not None:
            assert norm_w is not None and len(args) == 4
            p.flags |= ROPE_APPEND_FUSED
            p = MatvecRope(p, rope[0])
            args += list(rope[1])
        self.launch(MATVEC_KERNEL[ttype], with_peer(p, wait, push), args, (-(-n // 8), m, 1), variant)

    def peer_wait(self, slot: int, vector):
        """Waits (on the device, in stream order) for every rank's slice of exchange `slot` and fills in the plain
        floats of `vector` (a buffer inside the arena) for the host to read."""
        self.launch(EXT_PEER_WAIT, PeerExt(PEER_MAGIC, slot, PEER_NONE, 0), [vector], (1, 1, 1))

    def peer_next(self):
        """Ends a run of a launch list that uses exchanges: the epoch its tags derive from moves on."""
        self.launch(EXT_PEER_NEXT, PeerExt(PEER_MAGIC, PEER_NONE, PEER_NONE, 0), [], (1, 1, 1))

    def matmul(self, ttype, x, w, out, rows, n, k, col0=0, out_stride=None, accumulate=False, variant=0, layout=0):
        """The prefill multiply on half-precision weights. `variant` 0 is the exact f32 identity;
        VARIANT_PREFILL_TC is the tensor-core rung, where `layout` may say that x (X_HALF) and/or out (OUT_HALF)
        hold the weights' half type instead of f32."""
        p = MatmulBf16(rows, n, k, col0, out_stride if out_stride is not None else n, int(accumulate))
        p._pad[0] = layout
        self.launch(MATMUL_BF16 if ttype == "bf16" else MATMUL_F16, p, [x, w, out], (-(-n // 64), -(-rows // 16), 1), variant)

    # -- the quantised prefill family (src/plan/common.zig:389-477)
    def quantize_q8(self, x, qx, dx, rows, k, block, mode=0, eps=0.0, nw=None):
        """Rounds rows of activations to 8-bit blocks (block 256: Q8_K for the K-quants; 32: Q8_0). mode 1 rounds
        RMSNorm(x) * nw, mode 2 silu(gate) * up of rows gate | up."""
        self.launch(QUANTIZE_Q8, QuantizeQ8(k, block, mode, eps), [x, qx, dx, nw if nw is not None else x], (k // 256, rows, 1))

    def matmul_quant(self, ttype, qx, w, out, dx, rows, n, k, col0=0, out_stride=None, accumulate=False, k_slice=None,
                     slice_stride=0, variant=0):
        """`variant` VARIANT_PREFILL_TC (Q4_K only): the same integer arithmetic on tcgen05, sums in f32."""
        k_slice = k if k_slice is None else k_slice
        p = MatmulQuant(rows, n, k, col0, out_stride if out_stride is not None else n, int(accumulate), k_slice, slice_stride)
        self.launch(MATMUL_Q4_K if ttype == "q4_k" else MATMUL_Q8_0, p, [qx, w, out, dx],
                    (-(-n // 128), -(-rows // 32), -(-k // k_slice)), variant)

    def matmul_q8_0_float(self, x, w, out, rows, n, k, col0=0, out_stride=None, accumulate=False, k_slice=None, slice_stride=0):
        """Q8_0 weights against f32 activations as they are (no rounding): exact f32, k-ordered."""
        k_slice = k if k_slice is None else k_slice
        p = MatmulQuant(rows, n, k, col0, out_stride if out_stride is not None else n, int(accumulate), k_slice, slice_stride)
        self.launch(MATMUL_Q8_0_FLOAT, p, [x, w, out], (-(-n // 64), -(-rows // 16), -(-k // k_slice)))

    def matmul_reduce(self, partials, out, rows, n, slices, slice_stride, col0=0, out_stride=None, accumulate=False):
        p = MatmulReduce(rows, n, slices, col0, out_stride if out_stride is not None else n, int(accumulate), slice_stride, 0)
        self.launch(MATMUL_REDUCE, p, [partials, out], elementwise(rows * n))

    def rmsnorm(self, x, w, y, rows, dim, eps, w_rows=0):
        self.launch(RMSNORM, RmsNorm(rows, dim, eps, w_rows), [x, w, y], (rows, 1, 1))

    def silu_mul(self, gu, act, rows, width):
        self.launch(SILU_MUL, SiluMul(rows * width, width), [gu, act], elementwise(rows * width))

    def embed(self, ttype, tokens, w, out, m, dim, row0, chunk_rows, stride=0):
        self.launch(EMBED_KERNEL[ttype], Embed(dim, row0, chunk_rows, stride), [tokens, w, out], (m, 1, 1))

    def layout(self, ttype: str, src, dst, blocks: int):
        """File blocks -> the layout the multiplies read (Launcher.layout, kernels.zig): repack_q3_k for Q3_K, repad for
        the types whose blocks are padded."""
        if ttype == "q3_k":
            self.launch(REPACK_Q3_K, RepackQ3K(blocks), [src, dst], elementwise(blocks * 8))
        else:
            self.launch(REPAD, Repad(blocks, FILE_BLOCK[ttype], BLOCK_STRIDE[ttype], 0), [src, dst], elementwise(blocks * BLOCK_STRIDE[ttype] // 4))

    def repack_q8_0(self, src, dst, rows, k):
        self.launch(REPACK_Q8_0, RepackQ80(rows, k), [src, dst], elementwise(rows * row_bytes("q8_0", k) // 4))

    def rope_append(self, p: "RopeAppend", qkv, q_norm, k_norm, rope, kc, vc, step, m):
        self.launch(ROPE_APPEND, p, [qkv, q_norm, k_norm, rope, kc, vc, step], (p.heads + p.kv_heads, m, 1))

    def attn_split(self, p: "Attention", qg, kc, vc, part, step, keys, rows, variant=0):
        group = p.heads // p.kv_heads
        kern = ATTN_SPLIT if group <= ATTN_MAX_GROUP else ATTN_SPLIT_WIDE
        self.launch(kern, p, [qg, kc, vc, part, step], (p.kv_heads, -(-keys // ATTN_BLOCK), rows), variant)

    def attn_combine(self, p: "Attention", qg, part, out, step, rows):
        self.launch(ATTN_COMBINE, p, [qg, part, out, step], (p.heads, rows, 1))

    def delta_rule(self, p: "DeltaRule", conv, g, beta, state, out, step, proj=None, hist=None, kept=None, chunked_tokens=None,
                   chunk_variant=VARIANT_DELTA_CHUNK64):
        """The gated delta rule over a step. `chunked_tokens` = the step's token count selects the chunked form
        (64-token chunks, the remainder by the recurrent kernel; dim 128 only), which has no reference counterpart."""
        args = [conv, g, beta, state, out, step]
        if proj is not None:
            args += [proj, hist, kept]
        variant = 0
        if chunked_tokens is not None:
            p._pad = int(chunked_tokens)
            variant = chunk_variant
        self.launch(DELTA_RULE, p, args, (p.v_heads, -(-p.dim // 32), 1), variant)

    def delta_prep(self, p: "DeltaPrep", proj, conv_w, hist, out, dt_bias, a, g, beta, m):
        self.launch(DELTA_PREP, p, [proj, conv_w, hist, out, dt_bias, a, g, beta], (p.channels // p.head + 1, m, 1))

    def gated_norm(self, p: "GatedNorm", o, z, w, m):
        self.launch(GATED_NORM, p, [o, z, w], (p.v_heads, m, 1))

    def sample(self, s: "Sample", params_buf, logits, bias, prompt_mask, counts, work, state, nxt, step, steps=None):
        """One draw: every dispatch of kernels.sampleSteps, as the reference's host issues them."""
        for phase, rnd in (sample_steps(s) if steps is None else steps):
            groups = sample_groups(s.vocab) if phase in WIDE_PHASES else 1
            self.launch(SAMPLE, SamplePhase(phase, rnd), [logits, bias, prompt_mask, counts, work, state, nxt, step, params_buf],
                        (groups, 1, 1))

    def sample_unbump(self, s: "Sample", params_buf, logits, bias, prompt_mask, counts, work, state, nxt, step):
        self.launch(SAMPLE, SamplePhase(PH_UNBUMP, 0), [logits, bias, prompt_mask, counts, work, state, nxt, step, params_buf], (1, 1, 1))

    def mark_tokens(self, s: "Sample", tokens, mask):
        self.launch(MARK_TOKENS, s, [tokens, mask], elementwise(max(s.n_prompt, 1)))

    def draft(self, vocab: int, row: int, slot: int, logits, out):
        self.launch(DRAFT, Draft(vocab, row, slot, 0), [logits, out], (1, 1, 1))


def attention_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
