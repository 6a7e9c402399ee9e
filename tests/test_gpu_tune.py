"""The load-time sweep over the decode multiply's variants (the counterpart of src/tune/tune.zig): every candidate
agrees with the default within the sweep's tolerance, a diverging candidate is dropped, the table names a candidate
that exists, and a plan accepts the table."""
import numpy as np
import pytest

from zllm_b200 import kernels as K
from zllm_b200 import synth, tune

pytestmark = pytest.mark.gpu


def test_sweep_picks_an_agreeing_candidate_per_shape(gpu):
    rng = synth.rng_for("tune", "w")
    shapes = [("q4_k", 512, 1024), ("q8_0", 300, 1024), ("q8_0", 64, 96)]
    sweep = tune.Sweep(gpu, tokens=2)
    for ttype, n, k in shapes:
        raw = synth.q4_k_weights(rng, n, k) if ttype == "q4_k" else None
        if ttype == "q8_0":
            from zllm_b200 import model as M
            raw = M.split_q8_0_rows(synth.q8_0_weights(rng, n, k), k)
        sweep.add(ttype, gpu.put(raw), n, k)
        sweep.add(ttype, gpu.put(raw), n, k)  # a second matrix of the same shape is not tuned twice
    table = sweep.run()
    assert set(table) == set(shapes)
    assert sweep.dropped == 0
    for (ttype, n, k), v in table.items():
        assert v in [0] + K.MATVEC_CANDIDATES and K.matvec_variant_exists(ttype, k, v)
    timed = [r for r in sweep.report if r[4] is not None]
    assert len(timed) >= len(shapes) * 2 and all(r[4] > 0 for r in timed)
    # ragged Q8_0 rows (k = 96) only run on the scalar family
    assert all((r[3] == 0 or (r[3] >> 16) & 0xFF == K.FAMILY_SCALAR) for r in sweep.report if r[2] == 96)


def test_a_diverging_candidate_is_dropped(gpu, monkeypatch):
    rng = synth.rng_for("tune", "diverge")
    n, k = 128, 512
    sweep = tune.Sweep(gpu, tokens=1)
    sweep.add("q4_k", gpu.put(synth.q4_k_weights(rng, n, k)), n, k)
    real = sweep._batch
    bad = K.MATVEC_CANDIDATES[0]

    def batch(shape, variant, x, out):
        t = real(shape, variant, x, out)
        if variant == bad:  # spoil this candidate's output after it ran
            out.upload(np.full(n, 3.0, dtype=np.float32))
        return t

    monkeypatch.setattr(sweep, "_batch", batch)
    table = sweep.run()
    assert sweep.dropped == 1 and table[("q4_k", n, k)] != bad
