"""Parity of delta_prep, delta_rule and gated_norm with the CPU oracle (src/ref/qwen35.zig:425-563), through the
C ABI. Case designs follow src/kernels/check.zig:1807-2052."""
import numpy as np
import pytest

from tests.util import bits, rel_err, uniform
from zllm_b200 import kernels as K
from zllm_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-5


def run_delta(gpu, launcher, state, conv, g, beta, hk, hv, d, steps):
    """Runs the tokens as consecutive steps carrying the state; returns (state, out)."""
    ds = gpu.put(state)
    outs = []
    t0 = 0
    cd = conv.shape[1]
    for m in steps:
        out = gpu.zeros(m * hv * d * 4)
        step = gpu.put(np.array([m, t0, 0, 0], dtype=np.uint32))
        p = K.DeltaRule(hk, hv, d, cd, 1, cd, 0)
        launcher.delta_rule(p, gpu.put(conv[t0:t0 + m]), gpu.put(g[t0:t0 + m]), gpu.put(beta[t0:t0 + m]), ds, out, step)
        outs.append(out.download(np.float32).reshape(m, hv * d))
        t0 += m
    return ds.download(np.float32), np.concatenate(outs)


def test_delta_rule_two_steps_then_gated_norm(ref, gpu, launcher):
    # 4 value heads over 2 key heads, d = 128, 37 tokens as steps 20 + 17 carrying the state, then gated_norm.
    rng = np.random.default_rng(0x5EED)
    tokens, hk, hv, d = 37, 2, 4, 128
    conv, g, beta = synth.deltanet_inputs(rng, tokens, hk, hv, d, bf16=False)
    s0 = uniform(rng, (hv, d, d), 0.1)
    st, out = run_delta(gpu, launcher, s0, conv, g, beta, hk, hv, d, [20, 17])
    want_st, want_out = ref.delta_rule(s0, conv, g, beta, tokens, hk, hv, d, mode=ref.F64)
    assert rel_err(out, want_out) < TOL, rel_err(out, want_out)
    assert rel_err(st, want_st.ravel()) < TOL
    f32_st, f32_out = ref.delta_rule(s0, conv, g, beta, tokens, hk, hv, d)
    assert rel_err(out, f32_out) < 1e-3 and rel_err(st, f32_st.ravel()) < 1e-3
    # one 37-token step gives the same bits as 20 + 17
    st1, out1 = run_delta(gpu, launcher, s0, conv, g, beta, hk, hv, d, [37])
    assert np.array_equal(bits(out1), bits(out)) and np.array_equal(bits(st1), bits(st))
    # gated_norm on the result
    z = uniform(rng, (tokens, hv * d + 5), 2.0)
    nw = uniform(rng, d, 1.5)
    do = gpu.put(out)
    launcher.gated_norm(K.GatedNorm(hv, d, 1e-6, hv * d + 5, 5, 0), do, gpu.put(z), gpu.put(nw), tokens)
    got = do.download(np.float32).reshape(tokens, hv * d)
    want = ref.gated_norm(out, z[:, 5:].copy(), nw, tokens, hv, d, 1e-6)
    assert rel_err(got, want) < TOL


def test_config_deltanet_decode_on_seeded_state(ref, gpu, launcher):
    # Benchmark configuration: 16 heads, d = 128, bf16-valued q/k/v (q, k L2-normalised), one token on a state
    # produced by 64 oracle tokens.
    rng = synth.rng_for("cfg4", "decode")
    hk = hv = 16
    d = 128
    conv, g, beta = synth.deltanet_inputs(rng, 65, hk, hv, d, bf16=True)
    zero = np.zeros((hv, d, d), dtype=np.float32)
    seeded, _ = ref.delta_rule(zero, conv[:64], g[:64], beta[:64], 64, hk, hv, d)
    st, out = run_delta(gpu, launcher, seeded, conv[64:], g[64:], beta[64:], hk, hv, d, [1])
    want_st, want_out = ref.delta_rule(seeded, conv[64:], g[64:], beta[64:], 1, hk, hv, d, mode=ref.F64)
    assert rel_err(out, want_out) < TOL and rel_err(st, want_st.ravel()) < TOL
    f32_st, f32_out = ref.delta_rule(seeded, conv[64:], g[64:], beta[64:], 1, hk, hv, d)
    assert rel_err(out, f32_out) < 1e-3 and rel_err(st, f32_st.ravel()) < 1e-3


def test_delta_rule_long_sequence_from_zero(ref, gpu, launcher):
    # 512 tokens from a zero state in steps of 200/200/112 (states and outputs stay within 1e-3 of the f32 oracle).
    rng = synth.rng_for("cfg4", "prefill512")
    hk, hv, d, tokens = 2, 2, 128, 512
    conv, g, beta = synth.deltanet_inputs(rng, tokens, hk, hv, d, bf16=True)
    zero = np.zeros((hv, d, d), dtype=np.float32)
    st, out = run_delta(gpu, launcher, zero, conv, g, beta, hk, hv, d, [200, 200, 112])
    want_st, want_out = ref.delta_rule(zero, conv, g, beta, tokens, hk, hv, d, mode=ref.F64)
    assert rel_err(out, want_out) < 1e-4 and rel_err(st, want_st.ravel()) < 1e-4


def test_delta_prep_steps_with_history_and_keep(ref, gpu, launcher):
    # Steps of 5, 2, 1, 4 tokens with the conv history carried by delta_rule (check.zig:1807-1894), and the kept
    # state after row r (check.zig:1901-1959).
    rng = np.random.default_rng(31)
    hk, hv, d, taps, eps = 2, 4, 32, 4, 1e-6
    key_ch = 2 * hk * d
    channels = key_ch + hv * d
    inner = hv * d
    row = channels + inner + 2 * hv          # qkv | z | beta | alpha
    beta_off, alpha_off = channels + inner, channels + inner + hv
    total = 12
    proj = uniform(rng, (total, row), 1.0)
    conv_w = uniform(rng, (channels, taps), 0.5)
    dt_bias, a = uniform(rng, hv, 0.5), -np.abs(uniform(rng, hv, 1.0))
    want_conv = ref.conv_norm(proj[:, :channels].copy(), conv_w, total, hk, inner, d, taps, eps)
    want_beta = 1 / (1 + np.exp(-proj[:, beta_off:beta_off + hv].astype(np.float64)))
    xa = proj[:, alpha_off:alpha_off + hv].astype(np.float64) + dt_bias
    want_g = np.log1p(np.exp(xa)) * a
    s0 = np.zeros((hv, d, d), dtype=np.float32)
    want_state, want_out = ref.delta_rule(s0, want_conv, want_g.astype(np.float32), want_beta.astype(np.float32), total,
                                          hk, hv, d, mode=ref.F64)
    hist = gpu.zeros((taps - 1) * channels * 4)
    state = gpu.zeros(hv * d * d * 4)
    kept_hist = hv * d * d
    kept = gpu.zeros((kept_hist + (taps - 1) * channels) * 4)
    dcw, ddt, da = gpu.put(conv_w), gpu.put(dt_bias), gpu.put(a.astype(np.float32))
    t0 = 0
    outs = []
    for m, keep in [(5, 0), (2, 0), (1, 0), (4, 2)]:
        dproj = gpu.put(proj[t0:t0 + m])
        conv, g, beta = gpu.zeros(m * channels * 4), gpu.zeros(m * hv * 4), gpu.zeros(m * hv * 4)
        pp = K.DeltaPrep(channels, taps, key_ch, d, row, hv, beta_off, alpha_off, eps)
        launcher.delta_prep(pp, dproj, dcw, hist, conv, ddt, da, g, beta, m)
        got_conv = conv.download(np.float32).reshape(m, channels)
        assert rel_err(got_conv, want_conv[t0:t0 + m]) < TOL, (t0, rel_err(got_conv, want_conv[t0:t0 + m]))
        assert rel_err(beta.download(np.float32).reshape(m, hv), want_beta[t0:t0 + m]) < TOL
        assert rel_err(g.download(np.float32).reshape(m, hv), want_g[t0:t0 + m]) < TOL
        out = gpu.zeros(m * hv * d * 4)
        step = gpu.put(np.array([m, t0, 0, keep], dtype=np.uint32))
        pr = K.DeltaRule(hk, hv, d, channels, taps, row, kept_hist)
        launcher.delta_rule(pr, conv, g, beta, state, out, step, dproj, hist, kept)
        outs.append(out.download(np.float32).reshape(m, hv * d))
        if keep:
            # kept = the state and history as they stood after row keep - 1 of this step
            ks, _ = ref.delta_rule(s0, want_conv[:t0 + keep], want_g[:t0 + keep].astype(np.float32),
                                   want_beta[:t0 + keep].astype(np.float32), t0 + keep, hk, hv, d, mode=ref.F64)
            gk = kept.download(np.float32)
            assert rel_err(gk[:kept_hist], ks.ravel()) < TOL
            want_hist = proj[t0 + keep - (taps - 1):t0 + keep, :channels]
            assert np.array_equal(gk[kept_hist:].reshape(taps - 1, channels), want_hist)
        t0 += m
    assert rel_err(np.concatenate(outs), want_out) < TOL
    assert rel_err(state.download(np.float32), want_state.ravel()) < TOL
    # the history now holds the last taps-1 raw inputs, oldest first
    assert np.array_equal(hist.download(np.float32).reshape(taps - 1, channels), proj[total - (taps - 1):, :channels])
