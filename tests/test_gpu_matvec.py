"""Parity of the decode multiplies (matvec_q4_k / matvec_q8_0 / matvec_bf16 / matvec_f16) with the
CPU oracle, through the C ABI. Case designs follow the reference's kernel check
(src/kernels/check.zig:992-1113): odd output counts, NORM + ACCUMULATE from a random output, SILU_PAIR,
every variant, several x tiles, and bitwise equality of multi-token and single-token steps."""
import numpy as np
import pytest

from tests.util import bits, rel_err, split_q8_0, uniform
from zllm_b200 import kernels as K
from zllm_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 1e-5        # the reference's kernel-check tolerance (scale-relative, vs float64)
HARD_TOL = 1e-3   # the ceiling the benchmark configuration states, vs the f32 CPU reference

QUANT_VARIANTS = [0] + K.MATVEC_CANDIDATES


def make_weights(ref, ttype, rng, n, k, check_style=False):
    """Returns (device-layout bytes, oracle Matrix)."""
    if ttype == "q4_k":
        raw = synth.q4_k_weights(rng, n, k, 1e-4, 5e-2 if check_style else 1e-2, signed_scales=check_style)
        return raw, ref.Matrix(ref.Q4_K, raw, n, k)
    if ttype == "q8_0":
        raw = synth.q8_0_weights(rng, n, k, 1e-4, 5e-2 if check_style else 2e-3, signed_scales=check_style)
        return split_q8_0(raw, k), ref.Matrix(ref.Q8_0, raw, n, k)
    if ttype == "bf16":
        raw = synth.bf16_weights(rng, n, k, 0.05)
        return raw, ref.Matrix(ref.BF16, raw, n, k)
    raw = (rng.normal(0, 0.05, size=(n, k))).astype(np.float16)
    return raw.view(np.uint16), ref.Matrix(ref.F16, raw.view(np.uint16), n, k)


def truth(ref, x, mat, norm_w=None, eps=0.0):
    """float64 matvec over the oracle-decoded weights (check.zig:1033-1046)."""
    xs = x.astype(np.float64)
    if norm_w is not None:
        xs = np.stack([ref.rms_norm(r, norm_w, eps) for r in x]).astype(np.float64)
    return xs @ mat.dense().astype(np.float64).T


def variants_for(ttype, k=1024):
    if ttype == "q4_k":
        return QUANT_VARIANTS
    if ttype == "q8_0":
        # the tensor-core family takes Q8_0 rows of whole 128-weight tiles; the default falls back to scalar
        return QUANT_VARIANTS if k % 128 == 0 else [0, K.variant(0, 0, K.FAMILY_SCALAR)]
    return [0]


@pytest.mark.parametrize("ttype", ["q4_k", "q8_0", "bf16", "f16"])
def test_matvec_norm_accumulate_every_variant(ref, gpu, launcher, ttype):
    # 3 tokens x 100 outputs (a partial tile), k = 1024, NORM + ACCUMULATE from a random output.
    rng = np.random.default_rng(0x5EED)
    m, n, k, eps = 3, 100, 1024, 1e-6
    wbytes, mat = make_weights(ref, ttype, rng, n, k, check_style=True)
    x = uniform(rng, (m, k), 2.0)
    nw = uniform(rng, k, 1.5)
    start = uniform(rng, (m, n + 7), 1.0)
    want = start.astype(np.float64).copy()
    want[:, 3:3 + n] += truth(ref, x, mat, nw, eps)
    dx, dw, dn = gpu.put(x), gpu.put(wbytes), gpu.put(nw)
    singles = {}
    for v in variants_for(ttype):
        out = gpu.put(start)
        launcher.matvec(ttype, dx, dw, out, n, k, m=m, col0=3, out_stride=n + 7, flags=K.NORM | K.ACCUMULATE, eps=eps,
                        norm_w=dn, variant=v)
        got = out.download(np.float32).reshape(m, n + 7)
        assert rel_err(got, want) < TOL, (ttype, hex(v), rel_err(got, want))
        # columns outside [col0, col0 + n) are untouched
        assert np.array_equal(got[:, :3], start[:, :3]) and np.array_equal(got[:, 3 + n:], start[:, 3 + n:])
        # each token alone gives the same bits as inside the 3-token step
        for t in range(m):
            o1 = gpu.put(start[t:t + 1])
            launcher.matvec(ttype, gpu.put(x[t:t + 1]), dw, o1, n, k, m=1, col0=3, out_stride=n + 7,
                            flags=K.NORM | K.ACCUMULATE, eps=eps, norm_w=dn, variant=v)
            one = o1.download(np.float32)
            assert np.array_equal(bits(one), bits(got[t])), (ttype, hex(v), t)
        singles[v] = got
    # variants agree with the default within the tuning sweep's bar (rel L2 <= 1e-5, src/tune/tune.zig:171-183)
    for v, got in singles.items():
        d = got[:, 3:3 + n] - singles[0][:, 3:3 + n]
        assert np.linalg.norm(d) / np.linalg.norm(singles[0][:, 3:3 + n]) <= 1e-5


@pytest.mark.parametrize("ttype,k", [("q4_k", 4096), ("q8_0", 4160), ("q4_k", 14336), ("bf16", 4000)])
def test_matvec_silu_pair_and_tiles(ref, gpu, launcher, ttype, k):
    # Several x tiles, a tile tail (k = 4160), SILU_PAIR with gate and up rows in one matrix.
    rng = np.random.default_rng(k)
    m, pairs = 2, 75
    wbytes, mat = make_weights(ref, ttype, rng, 2 * pairs, k)
    x = synth.normal_f32(rng, m, k)
    full = truth(ref, x, mat)
    gate, up = full[:, :pairs], full[:, pairs:]
    want = gate / (1 + np.exp(-gate)) * up
    dx, dw = gpu.put(x), gpu.put(wbytes)
    for v in variants_for(ttype, k):
        out = gpu.zeros(m * pairs * 4)
        launcher.matvec(ttype, dx, dw, out, pairs, k, m=m, flags=K.SILU_PAIR, half=pairs, variant=v)
        got = out.download(np.float32).reshape(m, pairs)
        assert rel_err(got, want) < TOL, (ttype, hex(v), rel_err(got, want))


def test_matvec_x_stride_and_col_chunks(ref, gpu, launcher):
    # Inputs read out of wider rows (x_stride), outputs written as two row chunks of one matrix.
    rng = np.random.default_rng(77)
    m, n, k, wide = 4, 96, 512, 768
    wbytes, mat = make_weights(ref, "q4_k", rng, n, k)
    xw = synth.normal_f32(rng, m, wide)
    want = truth(ref, xw[:, :k].copy(), mat)
    dx = gpu.put(xw)
    rb = K.row_bytes("q4_k", k)
    dw = gpu.put(wbytes)
    out = gpu.zeros(m * n * 4)
    launcher.matvec("q4_k", dx, dw.at(0, 40 * rb), out, 40, k, m=m, col0=0, out_stride=n, x_stride=wide // 4)
    launcher.matvec("q4_k", dx, dw.at(40 * rb), out, n - 40, k, m=m, col0=40, out_stride=n, x_stride=wide // 4)
    got = out.download(np.float32).reshape(m, n)
    assert rel_err(got, want) < TOL


def test_config_q8_0_matvec_one_token(ref, gpu, launcher):
    # Benchmark configuration: x f32[1024] ~ N(0,1); W Q8_0 [3584 x 1024], q uniform in [-127,127],
    # d f16 uniform in [1e-4, 2e-3]; checked against the CPU reference's matmul.
    rng = synth.rng_for("cfg1", "w")
    n, k = 3584, 1024
    raw = synth.q8_0_weights(rng, n, k, 1e-4, 2e-3)
    x = synth.normal_f32(synth.rng_for("cfg1", "x"), 1, k)
    mat = ref.Matrix(ref.Q8_0, raw, n, k)
    want32 = ref.matmul(x, mat)
    want64 = ref.matmul(x, mat, mode=ref.F64)
    # the file layout goes through the load-time repack kernel, as the plan does
    src, dst = gpu.put(raw), gpu.zeros(n * K.row_bytes("q8_0", k))
    launcher.repack_q8_0(src, dst, n, k)
    assert np.array_equal(dst.download(np.uint8).reshape(n, -1), split_q8_0(raw, k))
    for v in QUANT_VARIANTS:
        out = gpu.zeros(n * 4)
        launcher.matvec("q8_0", gpu.put(x), dst, out, n, k, variant=v)
        got = out.download(np.float32)
        assert rel_err(got, want64[0]) < TOL, hex(v)
        assert np.abs(got - want32[0]).max() / np.abs(want32).max() < HARD_TOL


@pytest.mark.parametrize("batch", [1, 8])
def test_config_q4_k_ffn_up(ref, gpu, launcher, batch):
    # Benchmark configuration: x f32[batch, 4096] ~ N(0,1); W Q4_K [14336 x 4096]; out f32[batch, 14336].
    n, k = 14336, 4096
    raw = synth.q4_k_weights(synth.rng_for("cfg2", "w"), n, k, 1e-4, 1e-2)
    x = synth.normal_f32(synth.rng_for("cfg2", f"x{batch}"), batch, k)
    mat = ref.Matrix(ref.Q4_K, raw, n, k)
    want32 = ref.matmul(x, mat)
    want64 = ref.matmul(x, mat, mode=ref.F64)
    dw, dx = gpu.put(raw), gpu.put(x)
    outs = {}
    for v in QUANT_VARIANTS:
        out = gpu.zeros(batch * n * 4)
        launcher.matvec("q4_k", dx, dw, out, n, k, m=batch, variant=v)
        got = out.download(np.float32).reshape(batch, n)
        assert rel_err(got, want64) < TOL, (hex(v), rel_err(got, want64))
        assert np.abs(got - want32).max() / np.abs(want32).max() < HARD_TOL
        outs[v] = got
    if batch > 1:
        # every sequence of the batch equals its own single-token step, bit for bit
        for t in (0, batch - 1):
            o1 = gpu.zeros(n * 4)
            launcher.matvec("q4_k", gpu.put(x[t:t + 1]), dw, o1, n, k, m=1)
            assert np.array_equal(bits(o1.download(np.float32)), bits(outs[0][t]))


def test_embed_dequantises_bit_exactly(ref, gpu, launcher):
    # Dequantised weight values are the CPU reference's, bit for bit (golden blocks + random rows).
    from pathlib import Path

    g = np.load(Path(__file__).parent / "golden" / "dequant_gguf.npz")
    rng = np.random.default_rng(4)
    # Q4_K: rows of 3 super-blocks from the golden blocks
    rows4 = g["q4_k_bytes"].reshape(-1, 3 * 144)
    want4 = g["q4_k_f32_bits"].reshape(rows4.shape[0], 3 * 256)
    toks = np.arange(rows4.shape[0], dtype=np.uint32)[::-1].copy()
    out = gpu.zeros(toks.size * 768 * 4)
    launcher.embed("q4_k", gpu.put(toks), gpu.put(rows4), out, toks.size, 768, 0, rows4.shape[0])
    got = out.download(np.uint32).reshape(toks.size, 768)
    assert np.array_equal(got, want4[toks])
    # Q8_0: file layout (stride given) and split rows
    rows8 = g["q8_0_bytes"].reshape(-1, 8 * 34)
    want8 = g["q8_0_f32_bits"].reshape(rows8.shape[0], 256)
    toks = rng.permutation(rows8.shape[0]).astype(np.uint32)
    out = gpu.zeros(toks.size * 256 * 4)
    launcher.embed("q8_0", gpu.put(toks), gpu.put(rows8), out, toks.size, 256, 0, rows8.shape[0], stride=8 * 34)
    assert np.array_equal(out.download(np.uint32).reshape(toks.size, 256), want8[toks])
    out = gpu.zeros(toks.size * 256 * 4)
    launcher.embed("q8_0", gpu.put(toks), gpu.put(split_q8_0(rows8, 256)), out, toks.size, 256, 0, rows8.shape[0])
    assert np.array_equal(out.download(np.uint32).reshape(toks.size, 256), want8[toks])
    # random Q4_K rows against the oracle, and a chunk that only holds some of the tokens
    raw = synth.q4_k_weights(rng, 20, 1024, 1e-4, 5e-2, signed_scales=True)
    want = ref.dequantize(ref.Q4_K, raw, 20 * 1024).reshape(20, 1024)
    toks = np.array([3, 19, 0, 7, 12], dtype=np.uint32)
    out = gpu.put(np.full((5, 1024), 9.0, dtype=np.float32))
    launcher.embed("q4_k", gpu.put(toks), gpu.put(raw[5:15]), out, 5, 1024, 5, 10)
    got = out.download(np.float32).reshape(5, 1024)
    for i, tok in enumerate(toks):
        if 5 <= tok < 15:
            assert np.array_equal(bits(got[i]), bits(want[tok]))
        else:
            assert (got[i] == 9.0).all()  # tokens outside this chunk are left alone
