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


def test_the_sweep_times_a_shape_as_the_plan_uses_it_and_a_plan_takes_the_table(gpu):
    # A plan's own sweep: every shape of the model with its flags (norm prologue, SiLU pair), every layer's matrix in
    # turn; the table lands in the plan, and the tuned step gives the untuned step's logits within the sweep's bar.
    from zllm_b200 import model as M
    from zllm_b200.plan import DenseConfig, DenseProgram

    cfg = DenseConfig(layers=2, hidden=512, heads=8, kv_heads=2, head_dim=64, ff=1024, vocab=1536, max_ctx=192)
    weights = M.upload(M.host_model(cfg, "tune-plan"), cfg, gpu.put)

    def step(prog):
        prog.set_rope_table(gpu.put(DenseProgram.rope_table(cfg)))
        prog.write_step(np.array([7], dtype=np.uint32), np.array([33], dtype=np.uint32))
        prog.record_step(34)
        gpu.sync()
        return prog.logits.download(np.float32)

    plain = step(DenseProgram(gpu, cfg, weights, 1, gpu.zeros))
    prog = DenseProgram(gpu, cfg, weights, 1, gpu.zeros)
    table = prog.sweep()
    assert set(table) == {("q4_k", prog.qkv_row, 512), ("q4_k", 512, 512), ("q4_k", 1024, 512), ("q4_k", 512, 1024), ("q8_0", 1536, 512)}
    assert all(prog.variants[key] == v for key, v in table.items())
    tuned = step(prog)
    assert np.linalg.norm(tuned - plain) / np.linalg.norm(plain) <= 1e-5
    # the default and the best few of each shape tried inside the replayed step: four trials a shape, the default
    # first; a candidate stays only where it beat the default by the margin; same logits
    prog.write_step(np.array([7], dtype=np.uint32), np.array([33], dtype=np.uint32))
    refined = prog.refine(34, top=3, reps=2, margin=0.003)
    assert len(prog.refine_report) == len(table) and all(len(timed) == 4 for _, timed in prog.refine_report)
    for shape, timed in prog.refine_report:
        assert timed[0][1] == 0 and refined[shape] in [v for _, v in timed]
        assert refined[shape] == timed[DenseProgram.pick_trial([t for t, _ in timed], 0.003)][1]
    again = step(prog)
    assert np.linalg.norm(again - plain) / np.linalg.norm(plain) <= 1e-5


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
