"""The chunked gated delta rule against the sequential CPU oracle (src/ref/qwen35.zig:493-546 restated): the
chunked form is the same recurrence reassociated, so outputs and states must agree within 1e-3 of their scale.
Two arithmetics: the default runs the contractions on the tensor cores with every f32 operand as two bf16 terms
(measured ~1e-5 against the float64 oracle), the other is all f32 on the CUDA cores (~1e-6)."""
import numpy as np
import pytest

from zllm_b200 import abi
from zllm_b200 import kernels as K
from zllm_b200 import synth

from util import rel_err, uniform

pytestmark = pytest.mark.gpu


FORMS = [K.VARIANT_DELTA_CHUNK64, K.VARIANT_DELTA_CHUNK64_F32]


def run_chunked(gpu, launcher, state, conv, g, beta, hk, hv, d, steps, form=K.VARIANT_DELTA_CHUNK64):
    ds = gpu.put(state)
    outs, t0, cd = [], 0, conv.shape[1]
    for m in steps:
        out = gpu.zeros(m * hv * d * 4)
        step = gpu.put(np.array([m, t0, 0, 0], dtype=np.uint32))
        p = K.DeltaRule(hk, hv, d, cd, 1, cd, 0)
        launcher.delta_rule(p, gpu.put(conv[t0:t0 + m]), gpu.put(g[t0:t0 + m]), gpu.put(beta[t0:t0 + m]), ds, out, step,
                            chunked_tokens=m, chunk_variant=form)
        outs.append(out.download(np.float32).reshape(m, hv * d))
        t0 += m
    return ds.download(np.float32), np.concatenate(outs)


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("hk,hv,steps", [(2, 2, [64]), (2, 4, [300, 212]), (1, 3, [63, 65, 128])])
def test_chunked_matches_the_sequential_oracle(ref, gpu, launcher, hk, hv, steps, form):
    # one chunk; chunks with a recurrent tail (300 = 4 x 64 + 44) carrying the state across steps, two value
    # heads per key head; steps below, just above and at whole chunks. Starts from a random state.
    rng = synth.rng_for("cfg4", f"chunk-{hk}-{hv}-{steps}")
    d, tokens = 128, sum(steps)
    conv, g, beta = synth.deltanet_inputs(rng, tokens, hk, hv, d, bf16=True)
    s0 = uniform(rng, (hv, d, d), 0.1)
    st, out = run_chunked(gpu, launcher, s0, conv, g, beta, hk, hv, d, steps, form)
    want_st, want_out = ref.delta_rule(s0, conv, g, beta, tokens, hk, hv, d, mode=ref.F64)
    bar = 1e-4 if form == K.VARIANT_DELTA_CHUNK64 else 1e-5
    assert rel_err(out, want_out) < bar, rel_err(out, want_out)
    assert rel_err(st, want_st.ravel()) < bar, rel_err(st, want_st.ravel())
    f32_st, f32_out = ref.delta_rule(s0, conv, g, beta, tokens, hk, hv, d)
    assert rel_err(out, f32_out) < 1e-3 and rel_err(st, f32_st.ravel()) < 1e-3


@pytest.mark.parametrize("form", FORMS)
def test_slow_decay_keeps_long_memory(ref, gpu, launcher, form):
    # log-decays near zero (g = -0.01 softplus): the state carries hundreds of tokens, the triangular inverse
    # is far from the identity, and errors of early chunks are not forgotten.
    rng = synth.rng_for("cfg4", "slow-decay")
    hk, hv, d, tokens = 1, 2, 128, 512
    conv, g, beta = synth.deltanet_inputs(rng, tokens, hk, hv, d, bf16=True)
    g = (0.01 * g).astype(np.float32)
    zero = np.zeros((hv, d, d), dtype=np.float32)
    st, out = run_chunked(gpu, launcher, zero, conv, g, beta, hk, hv, d, [tokens], form)
    want_st, want_out = ref.delta_rule(zero, conv, g, beta, tokens, hk, hv, d, mode=ref.F64)
    assert rel_err(out, want_out) < 1e-3, rel_err(out, want_out)
    assert rel_err(st, want_st.ravel()) < 1e-3, rel_err(st, want_st.ravel())


@pytest.mark.parametrize("form", FORMS)
def test_named_layer_shape_prefill(ref, gpu, launcher, form):
    # batch 1, 4096 tokens, 16 heads of 128, q/k/v bf16 values, zero state: one step of 64 chunks.
    rng = synth.rng_for("cfg4", "prefill4096")
    hk, hv, d, tokens = 16, 16, 128, 4096
    conv, g, beta = synth.deltanet_inputs(rng, tokens, hk, hv, d, bf16=True)
    zero = np.zeros((hv, d, d), dtype=np.float32)
    st, out = run_chunked(gpu, launcher, zero, conv, g, beta, hk, hv, d, [tokens], form)
    want_st, want_out = ref.delta_rule(zero, conv, g, beta, tokens, hk, hv, d)
    assert rel_err(out, want_out) < 1e-3, rel_err(out, want_out)
    assert rel_err(st, want_st.ravel()) < 1e-3, rel_err(st, want_st.ravel())


def test_wrong_token_count_is_reported_not_guessed(gpu, launcher):
    # the host-side count must be the step's: the tail kernel refuses and the next sync reports it
    rng = synth.rng_for("cfg4", "mismatch")
    hk, hv, d, m = 1, 1, 128, 70
    conv, g, beta = synth.deltanet_inputs(rng, m, hk, hv, d, bf16=True)
    state, out = gpu.zeros(hv * d * d * 4), gpu.zeros(m * hv * d * 4)
    step = gpu.put(np.array([m - 1, 0, 0, 0], dtype=np.uint32))
    launcher.delta_rule(K.DeltaRule(hk, hv, d, conv.shape[1], 1, conv.shape[1], 0), gpu.put(conv), gpu.put(g), gpu.put(beta),
                        state, out, step, chunked_tokens=m)
    with pytest.raises(abi.ZcuError):
        gpu.sync()
