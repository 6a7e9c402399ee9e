"""Parity of the tensor-core prefill rung (tcgen05 / tensor memory) with the CPU oracle: activations rounded to
the weights' half type as the oracle rounds them (roundLikeLlama, src/ref/matmul.zig:228-258), f32 accumulation.
f32 outputs must agree to 1e-3 of the output scale (measured: ~1e-6); half outputs must be the oracle's value
rounded to the half type, give or take one unit in the last place where the two f32 sums straddle a tie."""
import numpy as np
import pytest

from zllm_b200 import kernels as K
from zllm_b200 import synth

from util import rel_err, uniform

pytestmark = pytest.mark.gpu

TC = K.VARIANT_PREFILL_TC


def _weights(rng, ttype, n, k, std):
    if ttype == "bf16":
        return synth.bf16_weights(rng, n, k, std)
    return rng.normal(0, std, size=(n, k)).astype(np.float16).view(np.uint16)


def _oracle(ref, ttype, x, raw, n, k):
    t = ref.BF16 if ttype == "bf16" else ref.F16
    return ref.matmul(ref.round_like_llama(t, x).reshape(x.shape), ref.Matrix(t, raw, n, k))


def _half_to_f32(ttype, bits):
    bits = np.asarray(bits, dtype=np.uint16)
    return synth.bf16_bits_to_f32(bits) if ttype == "bf16" else bits.view(np.float16).astype(np.float32)


def _to_half_bits(ttype, v):
    v = np.asarray(v, dtype=np.float32)
    return synth.to_bf16_bits(v) if ttype == "bf16" else v.astype(np.float16).view(np.uint16)


def test_rung_is_advertised(gpu):
    assert gpu.supports_prefill(0) and gpu.supports_prefill(TC)
    assert not gpu.supports_prefill(0xFFFF0000)  # the compensated rung does not exist here


@pytest.mark.parametrize("ttype", ["bf16", "f16"])
@pytest.mark.parametrize("rows,n,k", [(19, 100, 1024), (300, 520, 200), (128, 256, 64), (129, 272, 4096)])
def test_f32_in_f32_out(ref, gpu, launcher, ttype, rows, n, k):
    # token counts below, at and above a tile; n not a multiple of 16; a K tail (200 = 3 * 64 + 8)
    rng = synth.rng_for("matmul_tc", f"{ttype}-{rows}-{n}-{k}")
    raw = _weights(rng, ttype, n, k, 0.05)
    x = uniform(rng, (rows, k), 1.0)
    out = gpu.zeros(rows * n * 4)
    launcher.matmul(ttype, gpu.put(x), gpu.put(raw), out, rows, n, k, variant=TC)
    got = out.download(np.float32).reshape(rows, n)
    assert rel_err(got, _oracle(ref, ttype, x, raw, n, k)) < 1e-3


def test_weight_chunks_accumulate_at_odd_columns(ref, gpu, launcher):
    # two weight chunks accumulating onto a random output, the second at column 70 (no 16-byte stores there):
    # the reference's chunked-weights case (src/kernels/check.zig:311-333)
    rng = synth.rng_for("matmul_tc", "chunks")
    rows, n, k = 33, 150, 96
    raw = _weights(rng, "bf16", n, k, 0.05)
    x = uniform(rng, (rows, k), 1.0)
    start = uniform(rng, (rows, n), 1.0)
    out = gpu.put(start)
    dw, dx = gpu.put(raw), gpu.put(x)
    launcher.matmul("bf16", dx, dw.at(0, 70 * k * 2), out, rows, 70, k, col0=0, out_stride=n, accumulate=True, variant=TC)
    launcher.matmul("bf16", dx, dw.at(70 * k * 2), out, rows, 80, k, col0=70, out_stride=n, accumulate=True, variant=TC)
    want = start + _oracle(ref, "bf16", x, raw, n, k)
    assert rel_err(out.download(np.float32).reshape(rows, n), want) < 1e-3


def _check_half_out(ttype, got_bits, want_f32):
    """`got` is the half value nearest to a sum within 1e-5 of the output scale of the oracle's f32 sum."""
    want_bits = _to_half_bits(ttype, want_f32)
    assert (got_bits == want_bits).mean() > 0.99
    got = _half_to_f32(ttype, got_bits).astype(np.float64)
    want = want_f32.astype(np.float64)
    exp = np.floor(np.log2(np.maximum(np.abs(want), 1e-300)))
    spacing = np.exp2(exp - 7) if ttype == "bf16" else np.exp2(np.maximum(exp, -14) - 10)
    assert np.all(np.abs(got - want) <= 0.5 * spacing + 1e-5 * np.abs(want).max())


@pytest.mark.parametrize("ttype", ["bf16", "f16"])
def test_half_in_half_out(ref, gpu, launcher, ttype):
    rng = synth.rng_for("matmul_tc", f"half-{ttype}")
    rows, n, k = 200, 384, 512
    raw = _weights(rng, ttype, n, k, 0.02)
    xh = _to_half_bits(ttype, rng.normal(size=(rows, k)).astype(np.float32))
    out = gpu.zeros(rows * n * 2)
    launcher.matmul(ttype, gpu.put(xh), gpu.put(raw), out, rows, n, k, variant=TC, layout=K.X_HALF | K.OUT_HALF)
    got = out.download(np.uint16).reshape(rows, n)
    _check_half_out(ttype, got, _oracle(ref, ttype, _half_to_f32(ttype, xh), raw, n, k))


def test_named_prefill_shape_sampled_rows(ref, gpu, launcher):
    # 2048 tokens x 4096 x 4096, bf16 in and out, activations ~ N(0,1), weights ~ N(0, 0.02): two token rows
    # of every 128-row tile (every tile of the grid is touched) against the oracle over all 4096 outputs.
    rng = synth.rng_for("matmul_tc", "named")
    rows, n, k = 2048, 4096, 4096
    raw = synth.bf16_weights(rng, n, k, 0.02)
    xh = synth.to_bf16_bits(rng.normal(size=(rows, k)).astype(np.float32))
    out = gpu.zeros(rows * n * 2)
    launcher.matmul("bf16", gpu.put(xh), gpu.put(raw), out, rows, n, k, variant=TC, layout=K.X_HALF | K.OUT_HALF)
    got = out.download(np.uint16).reshape(rows, n)
    picks = np.array(sorted({128 * t + o for t in range(rows // 128) for o in (int(rng.integers(0, 128)), 127 - t % 7)}))
    want = _oracle(ref, "bf16", synth.bf16_bits_to_f32(xh[picks]), raw, n, k)
    _check_half_out("bf16", got[picks], want)
    # the rows not sampled are not zero and not wild: the whole output has the spread of N(0, 0.02 * sqrt(k))
    sd = float(synth.bf16_bits_to_f32(got).std())
    assert 1.1 < sd < 1.5
