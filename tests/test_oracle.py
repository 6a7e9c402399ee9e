"""Pins the CPU oracle (oracle/ref_cpu.cpp) to the reference's own known
answers for the hot path, and to the gguf-package dequantisation fixtures."""
import math
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).parent / "golden"


def bits(values):
    return np.asarray(values, dtype=np.float32).view(np.uint32)


def from_bits(words):
    return np.asarray(words, dtype=np.uint32).view(np.float32)


def test_rmsnorm_bit_fixture(ref):
    # src/ref/ops.zig:139-168, "RMSNorm matches pinned ggml arithmetic bitwise".
    x = from_bits([0xbf857c32, 0xbf8d2c0b, 0xbfa5eb34, 0x3ddf5988, 0xbdc29599, 0x3e230df4, 0xc10ccddd, 0x4052123d,
                   0xbf446fd1, 0xbf128c7d, 0xbe8b3a39, 0x3f1207f1, 0xbf78507a, 0x3d3ab508, 0x406c1281, 0x3e8f5b63,
                   0x3f2c4248])
    w = from_bits([0x3e9d12e6, 0x3f923ccb, 0xbf00548d, 0x3f07a020, 0x3f840c9f, 0x3f407d1a, 0xbfeefd55, 0xbf682ff8,
                   0x3e78a781, 0x3ea24f78, 0xbf9ced24, 0x3e55d151, 0x3fd00030, 0x3ffb9078, 0xbfab6e01, 0xbf50616f,
                   0x3fa4b9e8])
    want = [0xbe019766, 0xbeff32a0, 0x3e839a3d, 0x3cbb39dd, 0xbd1ecfe4, 0x3d41fd3a, 0x40cffc64, 0xbf96bc37,
            0xbd96f2c6, 0xbd930467, 0x3e070a0f, 0x3d40fcae, 0xbf1f9dac, 0x3d11269c, 0xbffa21fc, 0xbdb8a2bc,
            0x3eaf61ac]
    got = ref.rms_norm(x, w, 1e-5)
    assert bits(got).tolist() == want


def test_kv_f16_rounds_ties_to_even(ref):
    # src/ref/qwen35.zig:565-578.
    values = np.array([1.00048828125, 1.00146484375, -1.00048828125, -1.00146484375, 2.0 ** -25, 1.5 * 2.0 ** -24,
                       -(2.0 ** -25), 65504], dtype=np.float32)
    expected = np.array([1, 1.001953125, -1, -1.001953125, 0, 2.0 ** -23, -0.0, 65504], dtype=np.float32)
    assert bits(ref.f16_round(values)).tolist() == bits(expected).tolist()


def test_f16_converters_match_numpy_everywhere(ref):
    # Every binary16 pattern decodes as numpy does; a dense sample of f32 rounds as numpy does (IEEE RNE).
    lib = ref.lib()
    allh = np.arange(65536, dtype=np.uint16)
    want = allh.view(np.float16).astype(np.float32)
    got = np.array([lib.ref_f16_to_f32(int(h)) for h in allh], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(bits(got)[~nan], bits(want)[~nan]) and np.isnan(got[nan]).all()
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 2000), rng.normal(0, 3e4, 2000),
                        (np.arange(0, 2049) + 0.5) * 2.0 ** -24, [65519.9, 65520.0, 1e9, -1e9, 0.0]]).astype(np.float32)
    with np.errstate(over="ignore"):
        want16 = x.astype(np.float16).view(np.uint16)
    got16 = np.array([lib.ref_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got16, want16)


def test_dequantize_f32_f16_bf16(ref):
    # src/ref/tensor.zig:192-209.
    out = ref.dequantize(ref.F32, np.array([1.5, -2], dtype=np.float32).view(np.uint8), 2)
    assert out.tolist() == [1.5, -2]
    out = ref.dequantize(ref.F16, np.array([0.25, -65504], dtype=np.float16).view(np.uint8), 2)
    assert out.tolist() == [0.25, -65504]
    out = ref.dequantize(ref.BF16, np.array([0xC0, 0x3F, 0x00, 0xC0], dtype=np.uint8), 2)
    assert out.tolist() == [1.5, -2]
    with pytest.raises(ValueError):
        ref.dequantize(10, np.zeros(4, dtype=np.uint8), 2)  # q2_k: UnsupportedTensorType


def test_dequantize_matches_gguf_golden_bitwise(ref):
    g = np.load(GOLDEN / "dequant_gguf.npz")
    got8 = ref.dequantize(ref.Q8_0, g["q8_0_bytes"], g["q8_0_bytes"].shape[0] * 32)
    assert np.array_equal(bits(got8), g["q8_0_f32_bits"].ravel())
    got4 = ref.dequantize(ref.Q4_K, g["q4_k_bytes"], g["q4_k_bytes"].shape[0] * 256)
    assert np.array_equal(bits(got4), g["q4_k_f32_bits"].ravel())
    # the other block types of the loader path (src/ref/tensor.zig:54-181)
    for name, t in (("q3_k", ref.Q3_K), ("q5_k", ref.Q5_K), ("q6_k", ref.Q6_K), ("iq4_xs", ref.IQ4_XS)):
        by = g[f"{name}_bytes"]
        got = ref.dequantize(t, by, by.shape[0] * 256)
        assert np.array_equal(bits(got), g[f"{name}_f32_bits"].ravel()), name


def test_block_quantised_matrices_of_every_type_multiply_like_their_decoded_rows(ref):
    from zllm_b200 import synth

    rng = np.random.default_rng(9)
    x = rng.normal(size=(2, 512)).astype(np.float32)
    for name, t in (("q3_k", ref.Q3_K), ("q5_k", ref.Q5_K), ("q6_k", ref.Q6_K), ("iq4_xs", ref.IQ4_XS)):
        w = synth.kquant_weights(rng, name, 37, 512)
        m = ref.Matrix(t, w, 37, 512)
        dense = m.dense()
        assert np.array_equal(m.row(5), dense[5])
        want = x.astype(np.float64) @ dense.astype(np.float64).T
        got = ref.matmul(x, m, mode=ref.F64)
        assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max(), name


def test_q4_k_hand_built_block(ref):
    # Dyadic scales: every value is exact, so the layout can be checked by hand
    # (the reference's trick, src/ref/matmul.zig:351-352).
    b = np.zeros(144, dtype=np.uint8)
    b[0:2] = np.array([0.5], dtype=np.float16).view(np.uint8)
    b[2:4] = np.array([0.25], dtype=np.float16).view(np.uint8)
    sc = [1, 2, 3, 4, 33, 34, 35, 63]
    mn = [5, 6, 7, 8, 37, 38, 39, 62]
    s = b[4:16]
    for j in range(4):
        s[j] = sc[j] | ((sc[j + 4] >> 4) << 6)
        s[j + 4] = mn[j] | ((mn[j + 4] >> 4) << 6)
        s[j + 8] = (sc[j + 4] & 0xF) | ((mn[j + 4] & 0xF) << 4)
    qs = np.arange(128, dtype=np.uint8) * 7 + 3
    b[16:] = qs
    y = ref.dequantize(ref.Q4_K, b, 256)
    for sb in range(8):
        grp = qs[32 * (sb // 2):32 * (sb // 2) + 32]
        q = (grp & 0xF) if sb % 2 == 0 else (grp >> 4)
        want = (0.5 * sc[sb]) * q.astype(np.float32) - 0.25 * mn[sb]
        assert np.array_equal(y[32 * sb:32 * sb + 32], want.astype(np.float32))


def test_softplus_rope_norms(ref):
    lib = ref.lib()
    assert lib.ref_softplus(25.0) == 25.0  # linear above 20 (src/ref/ops.zig:57-60)
    assert abs(lib.ref_softplus(1.0) - math.log1p(math.e)) < 1e-6
    # src/ref/ops.zig:113-126
    x = np.arange(1, 9, dtype=np.float32)
    assert np.array_equal(ref.rope(x, 0, 4, 10000), x)
    r = ref.rope(x, 7, 4, 10000)
    assert abs(r[0] ** 2 + r[2] ** 2 - 10) < 1e-4 and abs(r[1] ** 2 + r[3] ** 2 - 20) < 1e-4
    assert np.array_equal(r[4:], x[4:])
    assert abs(r[0] - (math.cos(7) * 1 - math.sin(7) * 3)) < 1e-5
    # src/ref/ops.zig:128-137
    a = ref.l2_norm([3, 4, 0, 0], 0)
    assert abs(ref.dot(a, a) - 1) < 1e-6
    b = ref.rms_norm([2, -2], [1, 0.5], 0)
    assert abs(b[0] - 1) < 1e-6 and abs(b[1] + 0.5) < 1e-6
    # the rope table is the same formula (src/kernels/kernels.zig:730-744)
    t = ref.rope_table(9, 4, 10000).reshape(9, 2, 2)
    assert abs(t[7, 0, 0] - math.cos(7)) < 1e-6 and abs(t[7, 0, 1] - math.sin(7)) < 1e-6


def test_round_like_llama(ref):
    # src/ref/matmul.zig:394-419.
    x = np.zeros(256, dtype=np.float32)
    x[0] = 127
    x[1:7] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    x[7] = -0.1
    k = ref.round_like_llama(ref.Q4_K, x)
    assert k[1:7].tolist() == [0, 2, 2, 0, -2, -2]
    q8 = ref.round_like_llama(ref.Q8_0, x)
    assert q8[1:7].tolist() == [0, 2, 2, 0, -2, -2]
    assert bits(q8[7:8])[0] == 0
    y = np.zeros(32, dtype=np.float32)
    y[0] = from_bits([0x3f80000f])[0]
    y[1] = from_bits([0x3ca14298])[0]
    y[2] = -y[1]
    r = ref.round_like_llama(ref.Q8_0, y)
    d = np.float32(np.float16(y[0] / np.float32(127)))
    assert r[0] == np.float32(127) * d and r[1] == np.float32(2) * d and r[2] == np.float32(-2) * d
    # bf16: ties to even (src/ref/matmul.zig:250-255)
    v = from_bits([0x3f808000, 0x3f818000, 0x3f808001])
    assert bits(ref.round_like_llama(ref.BF16, v)).tolist() == [0x3f800000, 0x3f820000, 0x3f810000]


@pytest.mark.parametrize("threads", [1, 2, 7])
def test_matmul_matches_naive_for_every_remainder(ref, threads):
    # src/ref/matmul.zig:296-334.
    n, k, max_rows = 70, 37, 17
    rng = np.random.default_rng(1)
    x = (rng.random((max_rows, k), dtype=np.float32) - 0.5).astype(np.float32)
    w = (rng.random((n, k), dtype=np.float32) - 0.5).astype(np.float32)
    pool = ref.Pool(threads)
    m = ref.Matrix(ref.F32, w, n, k, pool)
    for j in range(n):
        assert np.array_equal(m.row(j), w[j])
    for rows in range(1, max_rows + 1):
        out = ref.matmul(x[:rows], m)
        want = np.zeros((rows, n), dtype=np.float32)
        for i in range(k):  # the naive f32 sum in i order
            want += np.outer(x[:rows, i], w[:, i]).astype(np.float32)
        assert np.abs(out - want).max() <= 1e-5
        assert np.array_equal(out, want)  # same order, same roundings
    pool.close()


def test_quantized_matrices_decode_panels_on_the_fly(ref):
    # src/ref/matmul.zig:336-380 (the Q8_0 arm; IQ4_XS is outside this path).
    n, k, rows = 70, 512, 9
    rng = np.random.default_rng(2)
    b = rng.integers(0, 256, size=(n * k // 32, 34), dtype=np.uint8)
    sc = np.where(np.arange(b.shape[0]) % 2 == 0, 0.0009765625, -0.0009765625).astype(np.float16)
    b[:, 0:2] = sc.view(np.uint8).reshape(-1, 2)
    w = ref.dequantize(ref.Q8_0, b, n * k).reshape(n, k)
    x = (rng.integers(-4, 5, size=(rows, k)) / 8).astype(np.float32)
    pool = ref.Pool(3)
    m = ref.Matrix(ref.Q8_0, b, n, k, pool)
    for j in (0, 32, n - 1):
        assert np.array_equal(m.row(j), w[j])
    out = ref.matmul(x, m)
    want = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(out - want).max() <= 1e-4
    for mode in (ref.FMA, ref.F64):
        assert np.abs(ref.matmul(x, m, mode=mode) - want).max() <= 1e-4
    pool.close()


def test_q4_k_matmul_modes_agree(ref):
    from zllm_b200 import synth

    n, k = 40, 1024
    rng = np.random.default_rng(5)
    wq = synth.q4_k_weights(rng, n, k)
    x = synth.normal_f32(rng, 3, k)
    m = ref.Matrix(ref.Q4_K, wq, n, k)
    w = m.dense().astype(np.float64)
    want = x.astype(np.float64) @ w.T
    scale = np.abs(want).max()
    for mode in (ref.MUL_ADD, ref.FMA, ref.F64):
        assert np.abs(ref.matmul(x, m, mode=mode) - want).max() / scale < 2e-6
    # llama.cpp-style activations differ, but only by the Q8_K rounding
    rounded = ref.matmul(x, m, act=True)
    assert 0 < np.abs(rounded - want).max() / scale < 2e-2


@pytest.mark.parametrize("style", ["neox", "normal"])
def test_attention_f16_kv_closed_form(ref, style):
    # src/ref/dense.zig:282-382: two tokens, one head of dim 2; K after RoPE and V
    # are rounded to binary16; token 0 sees itself, token 1 a two-way softmax.
    qw = np.array([[0.234567, 0.7654321], [-0.987654, 1.234567]], dtype=np.float32)
    kw = np.array([[0.3456789, -1.234567], [1.234567, 0.456789]], dtype=np.float32)
    vw = np.array([[1.00048828125, -0.33333334], [2.00146484375, 0.1234567]], dtype=np.float32)
    inp = np.eye(2, dtype=np.float32)
    scale = np.float32(1 / math.sqrt(2))
    rows_q = ref.matmul(inp, ref.Matrix(ref.F32, qw, 2, 2))
    rows_k = ref.matmul(inp, ref.Matrix(ref.F32, kw, 2, 2))
    rows_v = ref.matmul(inp, ref.Matrix(ref.F32, vw, 2, 2))
    norm = np.ones(2, dtype=np.float32)
    q, k = [], []
    for t in range(2):
        a, b = rows_q[t], rows_k[t]
        if style == "neox":
            a, b = ref.rms_norm(a, norm, 1e-5), ref.rms_norm(b, norm, 1e-5)
            a, b = ref.rope(a, t, 2, 10000), ref.rope(b, t, 2, 10000)
        else:
            a, b = ref.rope_normal(a, t, 2, 10000), ref.rope_normal(b, t, 2, 10000)
        q.append(a)
        k.append(b)
    kc = ref.to_f16_bits(np.stack(k))
    vc = ref.to_f16_bits(rows_v)
    k16 = kc.view(np.float16).astype(np.float32)
    v16 = vc.view(np.float16).astype(np.float32)
    out0 = ref.attend_decode(q[0], kc, vc, 1, 1, 1, 2, scale)[0]
    out1 = ref.attend_decode(q[1], kc, vc, 2, 1, 1, 2, scale)[0]
    assert np.abs(out0 - v16[0]).max() <= 1e-6
    s0, s1 = ref.dot(q[1], k16[0]) * scale, ref.dot(q[1], k16[1]) * scale
    mx = max(s0, s1)
    p0, p1 = math.exp(s0 - mx), math.exp(s1 - mx)
    want = (p0 * v16[0] + p1 * v16[1]) / (p0 + p1)
    assert np.abs(out1 - want).max() <= 1e-6
    # the f32 cache gives a different answer: rounding happened at the cache boundary
    assert not np.array_equal(v16, rows_v)


def test_attend_decode_gqa_matches_float64(ref):
    rng = np.random.default_rng(11)
    heads, kv_heads, hd, keys = 8, 2, 64, 150
    q = rng.normal(size=(heads, hd)).astype(np.float32)
    kc = rng.normal(size=(keys, kv_heads, hd)).astype(np.float16)
    vc = rng.normal(size=(keys, kv_heads, hd)).astype(np.float16)
    scale = 1 / math.sqrt(hd)
    got = ref.attend_decode(q, kc.view(np.uint16), vc.view(np.uint16), keys, heads, kv_heads, hd, scale)
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = kc[:, g].astype(np.float64) @ q[h].astype(np.float64) * scale
        p = np.exp(s - s.max())
        want = (p[:, None] * vc[:, g].astype(np.float64)).sum(0) / p.sum()
        assert np.abs(got[h] - want).max() / np.abs(want).max() < 1e-5


def test_delta_rule_f32_matches_float64_formula(ref):
    # The gated delta rule as src/kernels/check.zig:2018-2050 states it in float64.
    from zllm_b200 import synth

    rng = np.random.default_rng(7)
    tokens, hk, hv, d = 37, 2, 4, 32
    conv, g, beta = synth.deltanet_inputs(rng, tokens, hk, hv, d, bf16=False)
    s0 = (rng.normal(size=(hv, d, d)) * 0.1).astype(np.float32)
    S = s0.astype(np.float64)
    out = np.zeros((tokens, hv, d))
    key_dim = hk * d
    for t in range(tokens):
        for j in range(hv):
            q = conv[t, (j % hk) * d:(j % hk + 1) * d].astype(np.float64)
            k = conv[t, key_dim + (j % hk) * d:key_dim + (j % hk + 1) * d].astype(np.float64)
            v = conv[t, 2 * key_dim + j * d:2 * key_dim + (j + 1) * d].astype(np.float64)
            S[j] *= math.exp(g[t, j])
            delta = (v - S[j].T @ k) * beta[t, j]
            S[j] += np.outer(k, delta)
            out[t, j] = S[j].T @ q / math.sqrt(d)
    # two steps (20 + 17 tokens) carrying the state, as the reference's kernel check does
    st, o1 = ref.delta_rule(s0, conv[:20], g[:20], beta[:20], 20, hk, hv, d)
    st, o2 = ref.delta_rule(st, conv[20:], g[20:], beta[20:], 17, hk, hv, d)
    got = np.concatenate([o1, o2]).reshape(tokens, hv, d)
    assert np.abs(got - out).max() / np.abs(out).max() < 1e-5
    assert np.abs(st.reshape(hv, d, d) - S).max() / np.abs(S).max() < 1e-5
    st64, o64 = ref.delta_rule(s0, conv, g, beta, tokens, hk, hv, d, mode=ref.F64)
    assert np.abs(o64.reshape(tokens, hv, d) - out).max() / np.abs(out).max() < 1e-6


def test_gated_norm_and_conv_norm(ref):
    rng = np.random.default_rng(9)
    n, hv, d = 3, 2, 16
    o = rng.normal(size=(n, hv * d)).astype(np.float32)
    z = rng.normal(size=(n, hv * d)).astype(np.float32)
    w = rng.normal(size=d).astype(np.float32)
    got = ref.gated_norm(o, z, w, n, hv, d, 1e-6).reshape(n, hv, d)
    o64 = o.reshape(n, hv, d).astype(np.float64)
    z64 = z.reshape(n, hv, d).astype(np.float64)
    want = o64 / np.sqrt((o64 ** 2).mean(-1, keepdims=True) + 1e-6) * w * (z64 / (1 + np.exp(-z64)))
    assert np.abs(got - want).max() < 1e-5
    # conv: zero history, `kernel` taps, SiLU, then L2 norm of q and k heads
    hk, kernel = 1, 4
    cd = 2 * hk * d + hv * d
    qkv = rng.normal(size=(5, cd)).astype(np.float32)
    taps = rng.normal(size=(cd, kernel)).astype(np.float32)
    got = ref.conv_norm(qkv, taps, 5, hk, hv * d, d, kernel, 1e-6)
    pad = np.concatenate([np.zeros((kernel - 1, cd)), qkv.astype(np.float64)])
    want = np.zeros((5, cd))
    for t in range(5):
        s = (pad[t:t + kernel] * taps.T.astype(np.float64)).sum(0)
        want[t] = s / (1 + np.exp(-s))
        for i in range(2 * hk):
            seg = want[t, i * d:(i + 1) * d]
            want[t, i * d:(i + 1) * d] = seg / math.sqrt((seg ** 2).sum() + 1e-6)
    assert np.abs(got - want).max() < 1e-5
