"""The quantised prefill family against the CPU oracle: quantize_q8 rounds activations exactly as roundLikeLlama
does (src/ref/matmul.zig:203-258, bit for bit), and matmul_q4_k / matmul_q8_0 (+ matmul_reduce over k slices) give
the oracle's matmul on the rounded activations (the reference's Quant(t).matmul case, src/kernels/check.zig:839-871:
70 tokens x 150 outputs x 1024, whole and split over k, tolerance 1e-5)."""
import numpy as np
import pytest

from zllm_b200 import kernels as K
from zllm_b200 import model as M
from zllm_b200 import synth

from util import rel_err, uniform

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _quantize(gpu, launcher, x, block, mode=0, eps=0.0, nw=None, k=None):
    rows = x.shape[0]
    k = x.shape[1] if k is None else k
    qx, dx = gpu.zeros(rows * k), gpu.zeros(rows * (k // block) * 4)
    launcher.quantize_q8(gpu.put(x), qx, dx, rows, k, block, mode=mode, eps=eps, nw=None if nw is None else gpu.put(nw))
    gpu.sync()
    q = qx.download(np.int8).reshape(rows, k)
    d = dx.download(np.float32).reshape(rows, k // block)
    return qx, dx, q, d


@pytest.mark.parametrize("block,ttype", [(256, "q4_k"), (32, "q8_0")])
def test_quantize_q8_is_round_like_llama(ref, gpu, launcher, block, ttype):
    rng = synth.rng_for("quant-prefill", f"q{block}")
    rows, k = 5, 1024
    x = uniform(rng, (rows, k), 3.0)
    x[1, 256:512] = 0.0                       # an all-zero block: d = 0, q = 0
    x[2, 7] = x[2, 300] = 9.5                 # a tie for the largest value of two blocks: the first wins
    x[3, :32] = np.float32(1e-6)              # tiny values
    t = ref.Q4_K if ttype == "q4_k" else ref.Q8_0
    _, _, q, d = _quantize(gpu, launcher, x, block)
    got = q.astype(np.float32).reshape(rows, k // block, block) * d[:, :, None]
    want = ref.round_like_llama(t, x).reshape(rows, k // block, block)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.abs(q).max() <= 127


def test_quantize_q8_fuses_norm_and_silu(ref, gpu, launcher):
    rng = synth.rng_for("quant-prefill", "modes")
    rows, k, eps = 3, 512, 1e-6
    x = uniform(rng, (rows, k), 2.0)
    nw = (1 + 0.1 * rng.normal(size=k)).astype(np.float32)
    _, _, q, d = _quantize(gpu, launcher, x, 256, mode=1, eps=eps, nw=nw)
    normed = np.stack([ref.rms_norm(x[r], nw, eps) for r in range(rows)])
    want = ref.round_like_llama(ref.Q4_K, normed).reshape(rows, k // 256, 256)
    got = q.astype(np.float32).reshape(rows, k // 256, 256) * d[:, :, None]
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    gu = uniform(rng, (rows, 2 * k), 3.0)
    _, _, q, d = _quantize(gpu, launcher, gu, 32, mode=2, k=k)
    lib = ref.lib()
    act = np.array([[lib.ref_silu(float(g)) for g in row[:k]] for row in gu], dtype=np.float32) * gu[:, k:]
    want = ref.round_like_llama(ref.Q8_0, act).reshape(rows, k // 32, 32)
    got = q.astype(np.float32).reshape(rows, k // 32, 32) * d[:, :, None]
    assert rel_err(got, want) < 1e-6  # expf differs from the host's in the last place for a few gates


def _weights(rng, ttype, n, k):
    if ttype == "q4_k":
        raw = synth.q4_k_weights(rng, n, k)
        return raw, raw
    raw = synth.q8_0_weights(rng, n, k)
    return raw, M.split_q8_0_rows(raw, k)


@pytest.mark.parametrize("ttype", ["q4_k", "q8_0"])
def test_matmul_quant_whole_and_split_over_k(ref, gpu, launcher, ttype):
    rng = synth.rng_for("quant-prefill", f"mm-{ttype}")
    rows, n, k = 70, 150, 1024
    block = 256 if ttype == "q4_k" else 32
    raw, dev = _weights(rng, ttype, n, k)
    mat = ref.Matrix(ref.Q4_K if ttype == "q4_k" else ref.Q8_0, raw, n, k)
    x = uniform(rng, (rows, k), 1.0)
    want = ref.matmul(x, mat, act=True)
    qx, dx, _, _ = _quantize(gpu, launcher, x, block)
    dw = gpu.put(dev)
    out = gpu.zeros(rows * n * 4)
    launcher.matmul_quant(ttype, qx, dw, out, dx, rows, n, k)
    got = out.download(np.float32).reshape(rows, n)
    assert rel_err(got, want) < TOL, rel_err(got, want)
    # accumulate onto a random output, at a column offset of a wider row
    start = uniform(rng, (rows, n + 10), 1.0)
    out2 = gpu.put(start)
    launcher.matmul_quant(ttype, qx, dw, out2, dx, rows, n, k, col0=10, out_stride=n + 10, accumulate=True)
    got2 = out2.download(np.float32).reshape(rows, n + 10)
    assert rel_err(got2[:, 10:], start[:, 10:] + want) < TOL and np.array_equal(got2[:, :10], start[:, :10])
    # split over k into two slices, then matmul_reduce
    partials = gpu.zeros(2 * rows * n * 4)
    launcher.matmul_quant(ttype, qx, dw, partials, dx, rows, n, k, k_slice=512, slice_stride=rows * n)
    out3 = gpu.zeros(rows * n * 4)
    launcher.matmul_reduce(partials, out3, rows, n, 2, rows * n)
    assert rel_err(out3.download(np.float32).reshape(rows, n), want) < TOL
    # a step of fewer tokens than the buffers hold (the grid carries the count)
    out4 = gpu.zeros(rows * n * 4)
    p = K.MatmulQuant(rows, n, k, 0, n, 0, k, 0)
    launcher.launch(K.MATMUL_Q4_K if ttype == "q4_k" else K.MATMUL_Q8_0, p, [qx, dw, out4, dx], (2, 1, 1))
    got4 = out4.download(np.float32).reshape(rows, n)
    assert rel_err(got4[:32], want[:32]) < TOL and not got4[32:].any()


def test_matmul_q4_k_prefill_shape(ref, gpu, launcher):
    # 300 tokens x 512 outputs x 4096: several CTAs along both axes, 16 steps, partial last tiles
    rng = synth.rng_for("quant-prefill", "big")
    rows, n, k = 300, 520, 4096
    raw = synth.q4_k_weights(rng, n, k)
    x = rng.normal(size=(rows, k)).astype(np.float32)
    want = ref.matmul(x, ref.Matrix(ref.Q4_K, raw, n, k), act=True)
    qx, dx, _, _ = _quantize(gpu, launcher, x, 256)
    out = gpu.zeros(rows * n * 4)
    launcher.matmul_quant("q4_k", qx, gpu.put(raw), out, dx, rows, n, k)
    assert rel_err(out.download(np.float32).reshape(rows, n), want) < TOL


def test_matmul_q8_0_float_keeps_the_activations(ref, gpu, launcher):
    # Q8_0 weights against unrounded f32 activations: the oracle's exact matmul, every output summed in k order (so
    # a 3-token step equals the first rows of the 33-token step bit for bit), whole and split over k.
    rng = synth.rng_for("quant-prefill", "q8f")
    rows, n, k = 33, 150, 1024
    raw = synth.q8_0_weights(rng, n, k)
    dw = gpu.put(M.split_q8_0_rows(raw, k))
    x = uniform(rng, (rows, k), 1.0)
    want = ref.matmul(x, ref.Matrix(ref.Q8_0, raw, n, k))
    dxv = gpu.put(x)
    out = gpu.zeros(rows * n * 4)
    launcher.matmul_q8_0_float(dxv, dw, out, rows, n, k)
    got = out.download(np.float32).reshape(rows, n)
    assert rel_err(got, want) < TOL
    o3 = gpu.zeros(3 * n * 4)
    launcher.matmul_q8_0_float(gpu.put(x[:3]), dw, o3, 3, n, k)
    assert np.array_equal(o3.download(np.uint32).reshape(3, n), got[:3].view(np.uint32))
    partials = gpu.zeros(2 * rows * n * 4)
    launcher.matmul_q8_0_float(dxv, dw, partials, rows, n, k, k_slice=512, slice_stride=rows * n)
    out2 = gpu.put(np.ones((rows, n), dtype=np.float32))
    launcher.matmul_reduce(partials, out2, rows, n, 2, rows * n, accumulate=True)
    assert rel_err(out2.download(np.float32).reshape(rows, n), 1.0 + want) < TOL
