"""The sampler and FP8 oracles against the vectors the reference's own tests hold (src/sampler/sampler.zig:252-300,
src/ref/fp8.zig:64-86), and the host-side mirror of kernels.sampleSteps."""
import math

import numpy as np

from oracle import sampler as S
from zllm_b200 import kernels as K


def hist(n, prompt=()):
    m = np.zeros(n, dtype=bool)
    m[list(prompt)] = True
    return m, np.zeros(n, dtype=np.uint32)


def test_greedy_takes_the_first_maximum_after_bias_and_penalties():
    logits = np.array([1, 3, 3, 2.5], dtype=np.float32)
    prompt, counts = hist(4, prompt=[1])
    # token 1 is in the prompt: 3 / 1.5 = 2 < 3, so token 2 wins
    assert S.reference(logits, S.Params(temperature=0, repetition_penalty=1.5), prompt, counts, 0.5) == 2
    # a bias of +1 on token 3 makes it the maximum
    assert S.reference(logits, S.Params(temperature=0, logit_bias=[(3, 1.0)]), prompt, counts, 0.5) == 3
    # without either, ties go to the lower index
    assert S.reference(logits, S.Params(temperature=0), prompt, counts, 0.5) == 1


def test_top_p_keeps_tokens_while_the_mass_above_them_is_below_p():
    logits = np.log(np.array([0.5, 0.25, 0.125, 0.125])).astype(np.float32)
    prompt, counts = hist(4)
    assert S.reference(logits, S.Params(top_p=0.6), prompt, counts, 0.7) == 1
    assert S.reference(logits, S.Params(top_p=0.5), prompt, counts, 0.99) == 0
    assert S.reference(logits, S.Params(top_k=3), prompt, counts, 0.99) == 3      # tokens 2 and 3 tie at the third value
    assert S.reference(logits, S.Params(min_p=0.3), prompt, counts, 0.99) == 1    # drops p < 0.15


def test_validate_rejects_out_of_range_parameters_and_duplicate_biases():
    assert S.Params().validate(10)
    assert not S.Params(top_p=0).validate(10)
    assert not S.Params(temperature=-1).validate(10)
    assert not S.Params(logit_bias=[(1, 1.0), (1, 2.0)]).validate(10)
    assert not S.Params(logit_bias=[(10, 1.0)]).validate(10)


def test_deviation_is_zero_for_the_reference_draw_and_one_for_a_dropped_token():
    rng = np.random.default_rng(5)
    logits = (rng.normal(size=500) * 2).astype(np.float32)
    prompt, counts = hist(500)
    p = S.Params(temperature=0.7, top_k=40, top_p=0.9)
    for u in (0.0, 0.3, 0.999):
        tok = S.reference(logits, p, prompt, counts, u)
        assert S.deviation(logits, p, prompt, counts, u, tok, 1e-6) == 0.0
    assert S.deviation(logits, p, prompt, counts, 0.5, int(np.argmin(logits)), 1e-6) == 1.0


def test_fp8_every_finite_code_decodes_and_encodes_back_to_itself():
    for b in range(256):
        if b & 0x7F == 0x7F:
            continue
        assert S.fp8_encode(S.fp8_decode(b)) == b


def test_fp8_rounds_to_nearest_ties_to_even_and_clamps():
    d, e = S.fp8_decode, S.fp8_encode
    assert d(e(1000)) == 448 and d(e(-449)) == -448
    assert d(e(1.0625)) == 1 and d(e(1.1875)) == 1.25 and d(e(1.07)) == 1.125
    assert d(e(2.0 ** -10)) == 0 and d(e(3 * 2.0 ** -10)) == 2.0 ** -8
    assert d(e(2.0 ** -6 - 2.0 ** -12)) == 2.0 ** -6
    assert e(-0.0) == 0x80


def test_fp8_row_scale_is_the_smallest_power_of_two_that_fits():
    assert S.fp8_row_scale([0, -0.0]) == 1 and S.fp8_row_scale([448, -3]) == 1 and S.fp8_row_scale([449, 1]) == 2
    assert S.fp8_row_scale([-1.75]) == 2.0 ** -8 and S.fp8_row_scale([1.76]) == 2.0 ** -7


def test_sample_steps_mirror_the_reference_sequences():
    greedy = K.sample_params(32000, temperature=0.0)
    assert K.sample_steps(greedy) == [(K.PH_PREP, 0), (K.PH_REDUCE, 0)]
    small = K.sample_params(32000, temperature=0.7, top_k=40, top_p=0.9)
    assert len(K.sample_steps(small)) == 2 + 8 + 2 and K.sample_steps(small)[-1] == (K.PH_FINAL, 0)
    large = K.sample_params(32000, top_k=2000, top_p=0.8)
    assert len(K.sample_steps(large)) == 2 + 8 + 2 + 2 * 32 + 2          # kernels.max_sample_steps
    plain = K.sample_params(32000)
    assert K.sample_steps(plain) == [(K.PH_PREP, 0), (K.PH_REDUCE, 0), (K.PH_MASS, 0), (K.PH_PICK, 0)]
    assert K.sample_params(100, top_k=100).top_k == 0                    # top-k >= vocab disables it
    assert K.sample_state_words(32000) == 16 + 256 + 2 * 32 + 2048 and math.ceil(248320 / 1024) == K.sample_groups(248320)
