"""The tcgen05 forms of the Q4_K multiplies against the CPU oracle, through the C ABI: the tensor-core rung of
matmul_q4_k (variant 0xfffc0000; same bindings and parameter block as the integer-dot identity, the reference's
Quant(t).matmul case, src/kernels/check.zig:839-871) and the batched family of matvec_q4_k (up to 64 tokens in one
pass over the weights; case designs of src/kernels/check.zig:992-1113). Tolerance 1e-5 scale-relative."""
import numpy as np
import pytest

from zllm_b200 import kernels as K
from zllm_b200 import synth

from util import rel_err, uniform

pytestmark = pytest.mark.gpu
TOL = 1e-5
HARD_TOL = 1e-3
TC = K.VARIANT_PREFILL_TC
BATCHED = K.MATVEC_BATCHED


def _quantize(gpu, launcher, x):
    rows, k = x.shape
    qx, dx = gpu.zeros(rows * k), gpu.zeros(rows * (k // 256) * 4)
    launcher.quantize_q8(gpu.put(x), qx, dx, rows, k, 256)
    return qx, dx


def truth(ref, x, mat, norm_w=None, eps=0.0):
    xs = x.astype(np.float64)
    if norm_w is not None:
        xs = np.stack([ref.rms_norm(r, norm_w, eps) for r in x]).astype(np.float64)
    return xs @ mat.dense().astype(np.float64).T


def test_artifacts():
    from zllm_b200 import abi

    assert abi.artifact(K.MATMUL_Q4_K, TC) and not abi.artifact(K.MATMUL_Q8_0, TC)
    assert abi.artifact(K.MATVEC_KERNEL["q4_k"], BATCHED) and not abi.artifact(K.MATVEC_KERNEL["q8_0"], BATCHED)
    assert not abi.artifact(K.MATVEC_KERNEL["q4_k"], BATCHED | 2)


def test_matmul_q4_k_rung_whole_and_split_over_k(ref, gpu, launcher):
    rng = synth.rng_for("quant-tc", "mm")
    rows, n, k = 70, 150, 1024
    raw = synth.q4_k_weights(rng, n, k)
    x = uniform(rng, (rows, k), 1.0)
    want = ref.matmul(x, ref.Matrix(ref.Q4_K, raw, n, k), act=True)
    qx, dx = _quantize(gpu, launcher, x)
    dw = gpu.put(raw)
    out = gpu.zeros(rows * n * 4)
    launcher.matmul_quant("q4_k", qx, dw, out, dx, rows, n, k, variant=TC)
    got = out.download(np.float32).reshape(rows, n)
    assert rel_err(got, want) < TOL, rel_err(got, want)
    # the integer-dot identity gives the same values within the sums' f32 rounding
    ref_out = gpu.zeros(rows * n * 4)
    launcher.matmul_quant("q4_k", qx, dw, ref_out, dx, rows, n, k)
    assert rel_err(got, ref_out.download(np.float32).reshape(rows, n)) < 2e-6
    # accumulate onto a random output, at a column offset of a wider row
    start = uniform(rng, (rows, n + 10), 1.0)
    out2 = gpu.put(start)
    launcher.matmul_quant("q4_k", qx, dw, out2, dx, rows, n, k, col0=10, out_stride=n + 10, accumulate=True, variant=TC)
    got2 = out2.download(np.float32).reshape(rows, n + 10)
    assert rel_err(got2[:, 10:], start[:, 10:] + want) < TOL and np.array_equal(got2[:, :10], start[:, :10])
    # split over k into two slices, then matmul_reduce
    partials = gpu.zeros(2 * rows * n * 4)
    launcher.matmul_quant("q4_k", qx, dw, partials, dx, rows, n, k, k_slice=512, slice_stride=rows * n, variant=TC)
    out3 = gpu.zeros(rows * n * 4)
    launcher.matmul_reduce(partials, out3, rows, n, 2, rows * n)
    assert rel_err(out3.download(np.float32).reshape(rows, n), want) < TOL
    # a step of fewer tokens than the buffers hold (the grid carries the count)
    out4 = gpu.zeros(rows * n * 4)
    p = K.MatmulQuant(rows, n, k, 0, n, 0, k, 0)
    launcher.launch(K.MATMUL_Q4_K, p, [qx, dw, out4, dx], (2, 1, 1), TC)
    got4 = out4.download(np.float32).reshape(rows, n)
    assert rel_err(got4[:32], want[:32]) < TOL and not got4[32:].any()


def test_matmul_q4_k_rung_prefill_shape(ref, gpu, launcher):
    # 300 tokens x 520 outputs x 4096: several CTAs along both axes, 16 super-blocks, partial last tiles
    rng = synth.rng_for("quant-tc", "big")
    rows, n, k = 300, 520, 4096
    raw = synth.q4_k_weights(rng, n, k)
    x = rng.normal(size=(rows, k)).astype(np.float32)
    want = ref.matmul(x, ref.Matrix(ref.Q4_K, raw, n, k), act=True)
    qx, dx = _quantize(gpu, launcher, x)
    out = gpu.zeros(rows * n * 4)
    launcher.matmul_quant("q4_k", qx, gpu.put(raw), out, dx, rows, n, k, variant=TC)
    assert rel_err(out.download(np.float32).reshape(rows, n), want) < TOL


@pytest.mark.parametrize("m", [1, 3, 9, 40])
def test_matvec_batched_norm_accumulate(ref, gpu, launcher, m):
    # m tokens x 100 outputs (a partial tile), k = 1024, NORM + ACCUMULATE from a random output at a column offset.
    rng = np.random.default_rng(0x5EED + m)
    n, k, eps = 100, 1024, 1e-6
    raw = synth.q4_k_weights(rng, n, k, 1e-4, 5e-2, signed_scales=True)
    mat = ref.Matrix(ref.Q4_K, raw, n, k)
    x = uniform(rng, (m, k), 2.0)
    x[0, 256:512] = 0.0                    # an all-zero block
    x[m - 1, 3] = 1000.0                   # an outlier: the other values of its block keep 1e-5 of the OUTPUT scale
    nw = uniform(rng, k, 1.5)
    start = uniform(rng, (m, n + 7), 1.0)
    want = start.astype(np.float64).copy()
    want[:, 3:3 + n] += truth(ref, x, mat, nw, eps)
    out = gpu.put(start)
    launcher.matvec("q4_k", gpu.put(x), gpu.put(raw), out, n, k, m=m, col0=3, out_stride=n + 7, flags=K.NORM | K.ACCUMULATE,
                    eps=eps, norm_w=gpu.put(nw), variant=BATCHED)
    got = out.download(np.float32).reshape(m, n + 7)
    assert rel_err(got, want) < TOL, rel_err(got, want)
    assert np.array_equal(got[:, :3], start[:, :3]) and np.array_equal(got[:, 3 + n:], start[:, 3 + n:])
    # the default family agrees within the tuning sweep's bar (rel L2 <= 1e-5, src/tune/tune.zig:171-183)
    if m <= 4:
        out0 = gpu.put(start)
        launcher.matvec("q4_k", gpu.put(x), gpu.put(raw), out0, n, k, m=m, col0=3, out_stride=n + 7, flags=K.NORM | K.ACCUMULATE,
                        eps=eps, norm_w=gpu.put(nw))
        d = got - out0.download(np.float32).reshape(m, n + 7)
        assert np.linalg.norm(d) / np.linalg.norm(got) <= 1e-5


@pytest.mark.parametrize("k,half_gap", [(4096, 0), (14336, 53)])
def test_matvec_batched_silu_pair(ref, gpu, launcher, k, half_gap):
    # SILU_PAIR with gate and up rows in one matrix (`half_gap` rows of another tensor between them), several k slices.
    rng = np.random.default_rng(k)
    m, pairs = 8, 203
    rows = 2 * pairs + half_gap
    raw = synth.q4_k_weights(rng, rows, k)
    x = synth.normal_f32(rng, m, k)
    full = truth(ref, x, ref.Matrix(ref.Q4_K, raw, rows, k))
    gate, up = full[:, :pairs], full[:, pairs + half_gap:]
    want = gate / (1 + np.exp(-gate)) * up
    out = gpu.zeros(m * pairs * 4)
    launcher.matvec("q4_k", gpu.put(x), gpu.put(raw), out, pairs, k, m=m, flags=K.SILU_PAIR, half=pairs + half_gap, variant=BATCHED)
    got = out.download(np.float32).reshape(m, pairs)
    assert rel_err(got, want) < TOL, rel_err(got, want)


def test_matvec_batched_x_stride_and_col_chunks(ref, gpu, launcher):
    rng = np.random.default_rng(77)
    m, n, k, wide = 5, 296, 512, 768
    raw = synth.q4_k_weights(rng, n, k)
    xw = synth.normal_f32(rng, m, wide)
    want = truth(ref, xw[:, :k].copy(), ref.Matrix(ref.Q4_K, raw, n, k))
    dx, dw = gpu.put(xw), gpu.put(raw)
    rb = K.row_bytes("q4_k", k)
    out = gpu.zeros(m * n * 4)
    launcher.matvec("q4_k", dx, dw.at(0, 140 * rb), out, 140, k, m=m, col0=0, out_stride=n, x_stride=wide // 4, variant=BATCHED)
    launcher.matvec("q4_k", dx, dw.at(140 * rb), out, n - 140, k, m=m, col0=140, out_stride=n, x_stride=wide // 4, variant=BATCHED)
    assert rel_err(out.download(np.float32).reshape(m, n), want) < TOL


@pytest.mark.parametrize("batch", [8, 32])
def test_config_q4_k_ffn_up_batched(ref, gpu, launcher, batch):
    # Benchmark configuration: x f32[batch, 4096] ~ N(0,1); W Q4_K [14336 x 4096]; out f32[batch, 14336].
    n, k = 14336, 4096
    raw = synth.q4_k_weights(synth.rng_for("cfg2", "w"), n, k, 1e-4, 1e-2)
    x = synth.normal_f32(synth.rng_for("cfg2", f"x{batch}"), batch, k)
    mat = ref.Matrix(ref.Q4_K, raw, n, k)
    want32 = ref.matmul(x, mat)
    want64 = ref.matmul(x, mat, mode=ref.F64)
    out = gpu.zeros(batch * n * 4)
    launcher.matvec("q4_k", gpu.put(x), gpu.put(raw), out, n, k, m=batch, variant=BATCHED)
    got = out.download(np.float32).reshape(batch, n)
    assert rel_err(got, want64) < TOL, rel_err(got, want64)
    assert np.abs(got - want32).max() / np.abs(want32).max() < HARD_TOL


def test_matvec_batched_refuses_what_it_does_not_run(gpu, launcher):
    from zllm_b200 import abi

    k = 512
    w, x, out = gpu.zeros(8 * K.row_bytes("q4_k", k)), gpu.zeros(65 * k * 4), gpu.zeros(65 * 8 * 4)
    with pytest.raises(abi.ZcuError, match="at most 64"):
        launcher.matvec("q4_k", x, w, out, 8, k, m=65, variant=BATCHED)
    with pytest.raises(abi.ZcuError):
        launcher.matvec("q8_0", x, w, out, 8, k, m=8, variant=BATCHED)       # Q4_K only: no such artifact
    launcher.matvec("q4_k", x, w, out, 8, k, m=64, variant=BATCHED)           # the widest step: 128 columns
    gpu.sync()
    assert not out.download(np.float32).any()                                  # zero weights and activations
