"""The GPU sampler against the CPU oracle, case by case as the reference checks its own (src/kernels/check.zig:
2056-2127, 2586-2637): Gaussian logits (sigma 2) so every threshold cuts through a dense band, a random prompt mask
and output counts, seeded draws. Each token must be the oracle's draw up to rounding: `deviation` (the distance from
u to the token's CDF interval, with the min-p and top-p cuts allowed to move by the same relative amount) at most
1e-6 of the kept mass; greedy draws match exactly. Every trial also checks the stop flag, the next-step token, the
count bump and the processed logits left in `work` (bit-equal to the oracle's f32 operations)."""
import numpy as np
import pytest

from oracle import sampler as S
from zllm_b200 import kernels as K

pytestmark = pytest.mark.gpu
DRAW_TOLERANCE = 1e-6
TEST_BIAS = [(3, 9.0), (17, -50.0), (900, 4.5)]


def run_case(gpu, launcher, vocab, p: S.Params, trials, seed, all_phases=True):
    rng = np.random.default_rng(seed)
    logits = (rng.normal(size=vocab) * 2).astype(np.float32)
    prompt = rng.integers(0, 20, size=vocab) == 0
    counts = np.where(rng.integers(0, 30, size=vocab) == 0, 1 + rng.integers(0, 3, size=vocab), 0).astype(np.uint32)
    stops = [int(x) for x in rng.integers(0, vocab, size=3)]
    # make greedy and top-1 runs stop: the greedy token is a stop token
    stops[2] = S.reference(logits, S.Params(temperature=0, repetition_penalty=p.repetition_penalty, presence_penalty=p.presence_penalty,
                                            frequency_penalty=p.frequency_penalty, logit_bias=p.logit_bias), prompt, counts, 0)
    block = K.sample_params(vocab, float(p.temperature), p.top_k, float(p.top_p), float(p.min_p), float(p.repetition_penalty),
                            float(p.presence_penalty), float(p.frequency_penalty), len(p.logit_bias), stops)
    params = gpu.put(np.frombuffer(bytes(block), dtype=np.uint8))
    la, ba, pa = gpu.put(logits), gpu.put(p.bias_words()), gpu.put(prompt.astype(np.uint32))
    ca, work = gpu.zeros(vocab * 4), gpu.zeros(vocab * 4)
    state, nxt = gpu.zeros(K.sample_state_words(vocab) * 4), gpu.zeros(16)
    want_work = S.process(logits, p, prompt, counts)
    worst, exact = 0.0, 0
    for _ in range(trials):
        u = float(np.float32(rng.integers(0, 1 << 24)) * np.float32(2.0 ** -24))
        ca.upload(counts)
        step = gpu.put(np.array([1, 0, np.float32(u).view(np.uint32), 0], dtype=np.uint32))
        launcher.sample(block, params, la, ba, pa, ca, work, state, nxt, step, steps=None if all_phases else [(K.PH_PREP, 0)])
        gpu.sync()
        got, got_next, got_counts = state.download(np.uint32), nxt.download(np.uint32), ca.download(np.uint32)
        token = int(got[0])
        assert token < vocab and int(got[1]) == int(token in stops) and int(got_next[0]) == token
        assert int(got_counts[token]) == int(counts[token]) + 1 and int(got_counts.sum()) == int(counts.sum()) + 1
        assert np.array_equal(work.download(np.uint32), want_work.view(np.uint32))
        exact += token == S.reference(logits, p, prompt, counts, u)
        worst = max(worst, S.deviation(logits, p, prompt, counts, u, token, DRAW_TOLERANCE))
        # unbump undoes the draw's count
        launcher.sample_unbump(block, params, la, ba, pa, ca, work, state, nxt, step)
        gpu.sync()
        assert np.array_equal(ca.download(np.uint32), counts)
    return worst, exact


CASES = [
    ("greedy+penalties", 32000, S.Params(temperature=0, repetition_penalty=1.3, presence_penalty=0.5, frequency_penalty=0.2, logit_bias=TEST_BIAS), 4),
    ("k=40 p=0.9", 32000, S.Params(temperature=0.7, top_k=40, top_p=0.9), 16),
    ("min-p 0.05", 32000, S.Params(min_p=0.05), 16),
    ("top-p 0.5", 32000, S.Params(temperature=1.3, top_p=0.5), 16),
    ("T=1", 32000, S.Params(logit_bias=TEST_BIAS, repetition_penalty=1.1), 16),
    ("top-k 1", 32000, S.Params(top_k=1), 4),
    ("k=2000 p=0.8", 32000, S.Params(top_k=2000, top_p=0.8), 8),              # past the reference's candidate cap
    ("min-p 0.3 k=500", 32000, S.Params(min_p=0.3, top_k=500), 8),            # min-p leaves fewer than k: top-k removes nothing
    ("Qwen vocab", 248320, S.Params(temperature=0.8, top_k=20, top_p=0.95, min_p=0.01, repetition_penalty=1.05, presence_penalty=0.3), 3),
    ("Llama vocab", 128256, S.Params(temperature=0.6, top_p=0.9), 4),
    ("ragged vocab", 1000, S.Params(temperature=0.9, top_k=7, top_p=0.7), 8),
]


@pytest.mark.parametrize("name,vocab,p,trials", CASES, ids=[c[0] for c in CASES])
def test_draws_are_the_oracle_draws(gpu, launcher, name, vocab, p, trials):
    worst, exact = run_case(gpu, launcher, vocab, p, trials, seed=len(name) * 1000 + vocab)
    assert worst <= DRAW_TOLERANCE, (name, worst)
    if p.greedy or p.top_k == 1:
        assert exact == trials
    else:
        assert exact >= trials - 1, (name, exact)   # a draw within 1e-6 of a CDF boundary may land next door


def test_the_first_dispatch_alone_makes_the_draw(gpu, launcher):
    # the other phases of the reference's sequence launch nothing
    before = gpu.launch_count() if hasattr(gpu, "launch_count") else None
    worst, _ = run_case(gpu, launcher, 32000, S.Params(temperature=0.7, top_k=40, top_p=0.9), 2, seed=9, all_phases=False)
    assert worst <= DRAW_TOLERANCE
    del before


def test_ties_at_a_threshold_are_all_kept_and_draws_repeat(gpu, launcher):
    # 64 tokens share the largest value: top-k 3 keeps all of them; u walks through them in token order; the same u
    # gives the same token every time (integer masses: no dependence on the order of the sums)
    vocab = 5000
    logits = np.full(vocab, -3.0, dtype=np.float32)
    tied = np.arange(100, 100 + 64 * 7, 7)
    logits[tied] = 2.0
    block = K.sample_params(vocab, 1.0, 3, 1.0, 0.0)
    params = gpu.put(np.frombuffer(bytes(block), dtype=np.uint8))
    la, ba, pa = gpu.put(logits), gpu.put(np.zeros((1, 2), dtype=np.uint32)), gpu.zeros(vocab * 4)
    ca, work = gpu.zeros(vocab * 4), gpu.zeros(vocab * 4)
    state, nxt = gpu.zeros(K.sample_state_words(vocab) * 4), gpu.zeros(16)
    for k in (0, 1, 31, 63):
        u = np.float32((k + 0.5) / 64)
        seen = set()
        for _ in range(3):
            step = gpu.put(np.array([1, 0, u.view(np.uint32), 0], dtype=np.uint32))
            launcher.sample(block, params, la, ba, pa, ca, work, state, nxt, step)
            gpu.sync()
            seen.add(int(state.download(np.uint32)[0]))
        assert seen == {int(tied[k])}


def test_mark_tokens_and_draft(gpu, launcher):
    vocab = 3000
    rng = np.random.default_rng(3)
    toks = rng.integers(0, vocab, size=700).astype(np.uint32)
    block = K.sample_params(vocab, n_prompt=500)
    mask = gpu.zeros(vocab * 4)
    launcher.mark_tokens(block, gpu.put(toks), mask)
    gpu.sync()
    want = np.zeros(vocab, dtype=np.uint32)
    want[toks[:500]] = 1
    assert np.array_equal(mask.download(np.uint32), want)
    # draft: the first index of the maximum of the second of two rows; the maximum is planted twice
    rows = rng.normal(size=(2, vocab)).astype(np.float32)
    rows[1, 1234] = rows[1, 2999] = 9.0
    out = gpu.zeros(16)
    launcher.draft(vocab, vocab, 1, gpu.put(rows), out)
    gpu.sync()
    assert list(out.download(np.uint32)[:2]) == [0, 1234]
