"""Parity of rmsnorm, silu_mul, the exact prefill multiply and the command-stream path, through the C ABI."""
import numpy as np
import pytest

from tests.util import bits, rel_err, uniform
from zllm_b200 import abi, cmd
from zllm_b200 import kernels as K
from zllm_b200 import synth

pytestmark = pytest.mark.gpu


def test_rmsnorm_rows(ref, gpu, launcher):
    # 7 x 1000, tolerance 1e-6 (src/kernels/check.zig:267-285); the f64 sum makes it the oracle's bits.
    rng = np.random.default_rng(0x5EED)
    x, w = uniform(rng, (7, 1000), 3.0), uniform(rng, 1000, 1.5)
    y = gpu.zeros(7 * 1000 * 4)
    launcher.rmsnorm(gpu.put(x), gpu.put(w), y, 7, 1000, 1e-5)
    got = y.download(np.float32).reshape(7, 1000)
    want = np.stack([ref.rms_norm(r, w, 1e-5) for r in x])
    assert rel_err(got, want) < 1e-6
    assert (bits(got) == bits(want)).mean() > 0.999
    # the reference's own bit fixture (src/ref/ops.zig:139-168)
    xin = np.array([0xbf857c32, 0xbf8d2c0b, 0xbfa5eb34, 0x3ddf5988, 0xbdc29599, 0x3e230df4, 0xc10ccddd, 0x4052123d,
                    0xbf446fd1, 0xbf128c7d, 0xbe8b3a39, 0x3f1207f1, 0xbf78507a, 0x3d3ab508, 0x406c1281, 0x3e8f5b63,
                    0x3f2c4248], dtype=np.uint32)
    win = np.array([0x3e9d12e6, 0x3f923ccb, 0xbf00548d, 0x3f07a020, 0x3f840c9f, 0x3f407d1a, 0xbfeefd55, 0xbf682ff8,
                    0x3e78a781, 0x3ea24f78, 0xbf9ced24, 0x3e55d151, 0x3fd00030, 0x3ffb9078, 0xbfab6e01, 0xbf50616f,
                    0x3fa4b9e8], dtype=np.uint32)
    want_bits = [0xbe019766, 0xbeff32a0, 0x3e839a3d, 0x3cbb39dd, 0xbd1ecfe4, 0x3d41fd3a, 0x40cffc64, 0xbf96bc37,
                 0xbd96f2c6, 0xbd930467, 0x3e070a0f, 0x3d40fcae, 0xbf1f9dac, 0x3d11269c, 0xbffa21fc, 0xbdb8a2bc,
                 0x3eaf61ac]
    y = gpu.zeros(17 * 4)
    launcher.rmsnorm(gpu.put(xin), gpu.put(win), y, 1, 17, 1e-5)
    assert y.download(np.uint32).tolist() == want_bits


def test_silu_mul(ref, gpu, launcher):
    rng = np.random.default_rng(2)
    rows, width = 3, 333
    gu = uniform(rng, (rows, 2 * width), 4.0)
    act = gpu.zeros(rows * width * 4)
    launcher.silu_mul(gpu.put(gu), act, rows, width)
    g64, u64 = gu[:, :width].astype(np.float64), gu[:, width:].astype(np.float64)
    assert rel_err(act.download(np.float32).reshape(rows, width), g64 / (1 + np.exp(-g64)) * u64) < 1e-6


@pytest.mark.parametrize("ttype", ["bf16", "f16"])
def test_matmul_half_chunks_accumulate(ref, gpu, launcher, ttype):
    # 19 x 100 x 1024 whole, and 33 x 150 x 96 in two weight chunks accumulating onto a random output
    # (src/kernels/check.zig:288-333), tolerance 1e-5.
    rng = np.random.default_rng(0x5EED)

    def weights(n, k):
        if ttype == "bf16":
            raw = synth.bf16_weights(rng, n, k, 0.05)
            return raw, synth.bf16_bits_to_f32(raw)
        raw = rng.normal(0, 0.05, size=(n, k)).astype(np.float16)
        return raw.view(np.uint16), raw.astype(np.float32)

    rows, n, k = 19, 100, 1024
    raw, wf = weights(n, k)
    x = uniform(rng, (rows, k), 1.0)
    out = gpu.zeros(rows * n * 4)
    launcher.matmul(ttype, gpu.put(x), gpu.put(raw), out, rows, n, k)
    want = x.astype(np.float64) @ wf.astype(np.float64).T
    got = out.download(np.float32).reshape(rows, n)
    assert rel_err(got, want) < 1e-5
    mat = ref.Matrix(ref.BF16 if ttype == "bf16" else ref.F16, raw, n, k)
    assert rel_err(got, ref.matmul(x, mat)) < 1e-5
    # a 3-row step equals the first rows of the 19-row step, bit for bit
    o3 = gpu.zeros(3 * n * 4)
    launcher.matmul(ttype, gpu.put(x[:3]), gpu.put(raw), o3, 3, n, k)
    assert np.array_equal(bits(o3.download(np.float32)), bits(got[:3]).ravel())

    rows, n, k = 33, 150, 96
    raw, wf = weights(n, k)
    x = uniform(rng, (rows, k), 1.0)
    start = uniform(rng, (rows, n), 1.0)
    out = gpu.put(start)
    dw, dx = gpu.put(raw), gpu.put(x)
    launcher.matmul(ttype, dx, dw.at(0, 70 * k * 2), out, rows, 70, k, col0=0, out_stride=n, accumulate=True)
    launcher.matmul(ttype, dx, dw.at(70 * k * 2), out, rows, 80, k, col0=70, out_stride=n, accumulate=True)
    want = start + x.astype(np.float64) @ wf.astype(np.float64).T
    assert rel_err(out.download(np.float32).reshape(rows, n), want) < 1e-5


def test_command_stream_runs_a_matvec(ref, gpu):
    # The same multiply through zcu_execute: buffers, a parameter page, a bind group, a dispatch, a read.
    rng = np.random.default_rng(8)
    n, k, m = 64, 512, 2
    raw = synth.q4_k_weights(rng, n, k)
    x = synth.normal_f32(rng, m, k)
    want = x.astype(np.float64) @ ref.Matrix(ref.Q4_K, raw, n, k).dense().astype(np.float64).T
    r = cmd.Recorder()
    pipe = r.create_kernel(K.MATVEC_Q4_K, 0, 1 << 3, abi.artifact(K.MATVEC_Q4_K))
    bx, bw, bo = r.create_buffer(x.nbytes), r.create_buffer(raw.nbytes), r.create_buffer(m * n * 4)
    page = r.create_buffer(65536, cmd.UNIFORM | cmd.COPY_DST)
    params = np.zeros(65536, dtype=np.uint8)
    params[256:288] = np.frombuffer(bytes(K.Matvec(n, k, 0, n, 0.0, 0, 0, 0)), dtype=np.uint8)
    group = r.create_bind_group(pipe, [(0, page, 256, 32), (1, bx, 0, x.nbytes), (2, bw, 0, raw.nbytes),
                                       (3, bo, 0, m * n * 4), (4, bx, 0, 16)])
    # the dispatch is recorded BEFORE the writes: writes still land first (src/agility/host.zig:6-8)
    r.dispatch(pipe, (n // 8, m, 1), [group])
    r.write_buffer(bx, 0, x)
    r.write_buffer(bw, 0, raw)
    r.write_buffer(page, 0, params[:512])
    got = np.zeros((m, n), dtype=np.float32)
    r.read_buffer(7, bo, 0, got)
    r.submit(9)
    done = gpu.execute(r.batch())
    assert done == [(7, 0), (9, 0)]
    assert rel_err(got, want) < 1e-5
    # a second batch reuses the objects; destroy while work is pending is deferred to after the submit
    r.clear()
    r.clear_buffer(bo, 0, m * n * 4)
    r.dispatch(pipe, (n // 8, m, 1), [group])
    r.destroy(cmd.KIND_BUFFER, bo)
    got2 = np.zeros((m, n), dtype=np.float32)
    r.read_buffer(1, bo, 0, got2)
    r.submit(2)
    assert gpu.execute(r.batch()) == [(1, 0), (2, 0)]
    assert np.array_equal(got2, got)
    r.clear()
    r.clear_buffer(bo, 0, 4)
    with pytest.raises(abi.ZcuError) as e:
        gpu.execute(r.batch())
    assert e.value.name == "BadId"


def test_profile_and_graph_replay(ref, gpu, launcher):
    rng = np.random.default_rng(9)
    n, k = 128, 1024
    raw = synth.q4_k_weights(rng, n, k)
    x = synth.normal_f32(rng, 1, k)
    dw, dx, out = gpu.put(raw), gpu.put(x), gpu.zeros(n * 4)
    launcher.matvec("q4_k", dx, dw, out, n, k)
    first = out.download(np.float32)
    out.zero()
    gpu.sync()
    gpu.capture_begin()
    launcher.matvec("q4_k", dx, dw, out, n, k)
    launcher.matvec("q4_k", dx, dw, out, n, k, flags=K.ACCUMULATE)
    graph = gpu.capture_end()
    assert not out.download(np.float32).any()  # capturing ran nothing
    gpu.graph_launch(graph)
    gpu.sync()
    assert np.array_equal(out.download(np.float32), first + first)
