"""One decode step of a small Llama-shaped Q4_K model through the plan's launch list, against the CPU oracle's
layer-by-layer restatement of src/ref/dense.zig (each sequence on its own, shared weights)."""
import numpy as np
import pytest

from tests.util import rel_err, rel_l2
from zllm_b200 import kernels as K
from zllm_b200 import model as M
from zllm_b200.plan import DenseConfig, DenseProgram

pytestmark = pytest.mark.gpu

CFG = DenseConfig(layers=3, hidden=512, heads=8, kv_heads=2, head_dim=64, ff=1024, vocab=1536, rope_base=500000.0,
                  eps=1e-5, max_ctx=320)


def oracle_step(ref, cfg, host, token, pos, kc, vc):
    """Logits of one sequence: embedding row, every layer on the sequence's cache, output norm + head."""
    e, hd = cfg.hidden, cfg.head_dim
    x = ref.dequantize(ref.Q4_K, host["embed"][token], e)
    for il, lw in enumerate(host["layers"]):
        rows = lw["wqkv"]
        layer = {
            "attn_norm": lw["attn_norm"], "ffn_norm": lw["ffn_norm"],
            "wq": ref.Matrix(ref.Q4_K, rows[:cfg.q_dim], cfg.q_dim, e),
            "wk": ref.Matrix(ref.Q4_K, rows[cfg.q_dim:cfg.q_dim + cfg.kv_dim], cfg.kv_dim, e),
            "wv": ref.Matrix(ref.Q4_K, rows[cfg.q_dim + cfg.kv_dim:], cfg.kv_dim, e),
            "wo": ref.Matrix(ref.Q4_K, lw["wo"], e, cfg.q_dim),
            "gate": ref.Matrix(ref.Q4_K, lw["wgu"][:cfg.ff], cfg.ff, e),
            "up": ref.Matrix(ref.Q4_K, lw["wgu"][cfg.ff:], cfg.ff, e),
            "down": ref.Matrix(ref.Q4_K, lw["wdown"], e, cfg.ff),
        }
        x = ref.dense_decode_layer(layer, x, kc[il], vc[il], pos, cfg.heads, cfg.kv_heads, hd, cfg.ff, cfg.eps,
                                   cfg.rope_base, K.attention_scale(hd))
    head = ref.Matrix(ref.Q8_0, host["head"], cfg.vocab, e)
    return ref.dense_head(x, host["out_norm"], head, cfg.eps), x


@pytest.mark.parametrize("batch", [1, 3, 6])
def test_decode_step_matches_oracle(ref, gpu, batch):
    cfg = CFG
    host = M.host_model(cfg, "tiny")
    weights = M.upload(host, cfg, gpu.put)
    prog = DenseProgram(gpu, cfg, weights, batch, gpu.zeros)
    prog.set_rope_table(gpu.put(DenseProgram.rope_table(cfg)))
    assert np.array_equal(DenseProgram.rope_table(cfg), ref.rope_table(cfg.max_ctx, cfg.head_dim, cfg.rope_base))
    rng = np.random.default_rng(batch)
    positions = np.array([150, 7, 299, 0, 64, 201][:batch], dtype=np.uint32)
    tokens = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    # a cache of N(0,1) f16 values before each sequence's position
    kv_shape = (batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim)
    kc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    vc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    for il in range(cfg.layers):
        prog.kc[il].upload(kc_host[il].view(np.uint16))
        prog.vc[il].upload(vc_host[il].view(np.uint16))
    prog.write_step(tokens, positions)
    prog.record_step(int(positions.max()) + 1)
    gpu.sync()
    logits = prog.logits.download(np.float32).reshape(batch, cfg.vocab)
    hidden = prog.x.download(np.float32).reshape(batch, cfg.hidden)
    # (six sequences: the Q4_K multiplies take the batched family - columns, multiply, reduction)
    assert prog.batched == (batch == 6)
    assert prog.launches_per_step == 1 + (7 - prog.fuse_rope + 8 * prog.batched) * cfg.layers + 1
    for b in range(batch):
        kc = [np.ascontiguousarray(kc_host[il][b]).view(np.uint16).copy() for il in range(cfg.layers)]
        vc = [np.ascontiguousarray(vc_host[il][b]).view(np.uint16).copy() for il in range(cfg.layers)]
        want_logits, want_x = oracle_step(ref, cfg, host, int(tokens[b]), int(positions[b]), kc, vc)
        # the reference's model-tier bounds for a decode step: rel-L2 <= 1e-4, cosine >= 0.999999
        assert rel_l2(hidden[b], want_x) < 1e-4, (b, rel_l2(hidden[b], want_x))
        assert rel_l2(logits[b], want_logits) < 1e-4
        cos = float(np.dot(logits[b], want_logits) / (np.linalg.norm(logits[b]) * np.linalg.norm(want_logits)))
        assert cos > 0.999999
        assert int(np.argmax(logits[b])) == int(np.argmax(want_logits))
        # the step appended this token's K and V (f16, RNE) at its position, and nothing else
        p = int(positions[b])
        for il in (0, cfg.layers - 1):
            got_k = prog.kc[il].download(np.uint16).reshape(kv_shape)[b]
            want_k = kc[il].reshape(cfg.max_ctx, cfg.kv_heads, cfg.head_dim)[p]
            # (f16 roundings of f32 values that agree to 1e-6: the same bits, or rarely neighbours)
            assert np.abs(got_k[p].view(np.int16).astype(np.int32) - want_k.view(np.int16).astype(np.int32)).max() <= 1
            assert np.mean(got_k[p] == want_k) > 0.99
            mask = np.ones(cfg.max_ctx, dtype=bool)
            mask[p] = False
            assert np.array_equal(got_k[mask], kc_host[il][b].view(np.uint16)[mask])


def test_decode_step_graph_replay_and_batch_rows_are_independent(ref, gpu):
    # A captured step replays with new tokens/positions written to the step buffers, and every sequence of a
    # batch equals the same sequence run alone, bit for bit.
    cfg = CFG
    host = M.host_model(cfg, "tiny")
    weights = M.upload(host, cfg, gpu.put)
    rng = np.random.default_rng(5)
    batch = 4
    positions = np.array([40, 41, 100, 5], dtype=np.uint32)
    tokens = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    kv_shape = (batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim)
    kc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    vc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]

    def run(seqs, graph):
        b = len(seqs)
        prog = DenseProgram(gpu, cfg, weights, b, gpu.zeros)
        prog.set_rope_table(gpu.put(DenseProgram.rope_table(cfg)))
        for il in range(cfg.layers):
            prog.kc[il].upload(np.ascontiguousarray(kc_host[il][seqs]).view(np.uint16))
            prog.vc[il].upload(np.ascontiguousarray(vc_host[il][seqs]).view(np.uint16))
        prog.write_step(tokens[seqs], positions[seqs])
        if graph:
            gpu.sync()
            gpu.capture_begin()
            prog.record_step(cfg.max_ctx)
            g = gpu.capture_end()
            gpu.graph_launch(g)
        else:
            prog.record_step(int(positions[seqs].max()) + 1)
        gpu.sync()
        return prog.logits.download(np.float32).reshape(b, cfg.vocab)

    whole = run([0, 1, 2, 3], graph=True)
    for s in range(batch):
        alone = run([s], graph=False)
        assert np.array_equal(alone[0].view(np.uint32), whole[s].view(np.uint32)), s


@pytest.mark.parametrize("batch", [1, 2, 4])
def test_rope_append_in_the_multiply_epilogue_equals_its_own_launch(gpu, batch):
    # rope_append fused into the Q|K|V multiply (one launch fewer per layer) gives the same rotated queries,
    # the same cache rows and the same logits as the separate kernel, bit for bit.
    cfg = CFG
    host = M.host_model(cfg, "tiny")
    weights = M.upload(host, cfg, gpu.put)
    rng = np.random.default_rng(23 + batch)
    positions = np.array([150, 7, 299, 64][:batch], dtype=np.uint32)
    tokens = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    kv_shape = (batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim)
    kc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    vc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    got = {}
    for fuse in (False, True):
        prog = DenseProgram(gpu, cfg, weights, batch, gpu.zeros, fuse_rope=fuse)
        prog.set_rope_table(gpu.put(DenseProgram.rope_table(cfg)))
        for il in range(cfg.layers):
            prog.kc[il].upload(kc_host[il].view(np.uint16))
            prog.vc[il].upload(vc_host[il].view(np.uint16))
        prog.write_step(tokens, positions)
        prog.record_step(int(positions.max()) + 1)
        gpu.sync()
        got[fuse] = ([prog.logits.download(np.uint32), prog.qkv.download(np.uint32), prog.x.download(np.uint32)]
                     + [c.download(np.uint16) for c in prog.kc + prog.vc])
    for a, b in zip(got[False], got[True]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("batch", [1, 2])
def test_peer_exchange_with_one_rank_equals_the_plain_step(gpu, batch):
    # The tensor-parallel path with a world of one: outputs go through the arena, every producer publishes its
    # exchange slot and every consumer waits for it (its own count). Same bits as the plain step, also when the
    # step is captured once and replayed (the counters keep growing).
    from zllm_b200 import abi

    cfg = CFG
    host = M.host_model(cfg, "tiny")
    weights = M.upload(host, cfg, gpu.put)
    rng = np.random.default_rng(77)
    kv_shape = (batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim)
    kc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    vc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    arena = abi.PeerArena(gpu, 0, 1, DenseProgram.arena_bytes(cfg, batch), DenseProgram.arena_slots(cfg))

    def fresh(**kw):
        prog = DenseProgram(gpu, cfg, weights, batch, gpu.zeros, **kw)
        prog.set_rope_table(gpu.put(DenseProgram.rope_table(cfg)))
        for il in range(cfg.layers):
            prog.kc[il].upload(kc_host[il].view(np.uint16))
            prog.vc[il].upload(vc_host[il].view(np.uint16))
        return prog

    plain, peer = fresh(), fresh(arena=arena)
    graph = None
    for token, pos in [(5, 100), (900, 101), (31, 102)]:
        tok = (np.arange(batch, dtype=np.uint32) * 37 + token) % cfg.vocab
        ps = np.array([pos + 11 * s for s in range(batch)], dtype=np.uint32)
        plain.write_step(tok, ps)
        plain.record_step(cfg.max_ctx)
        peer.write_step(tok, ps)
        if graph is None:
            gpu.sync()
            gpu.capture_begin()
            peer.record_step(cfg.max_ctx)
            graph = gpu.capture_end()
        gpu.graph_launch(graph)
        gpu.sync()
        for name in ("logits", "x", "att", "act"):
            assert np.array_equal(getattr(plain, name).download(np.uint32), getattr(peer, name).download(np.uint32)), (name, pos)


@pytest.mark.parametrize("batch", [1, 8])
def test_one_layer_at_the_benchmark_shape_matches_oracle(ref, gpu, batch):
    # The shapes the decode benchmark times (hidden 4096, SwiGLU 14336, 32 query / 8 KV heads of 128, 128256-row Q8_0
    # head, f16 cache at position 8192), one layer deep: the step against the oracle's layer and head, per sequence.
    # (batch 8: the Q4_K multiplies take the batched family, the head runs in passes of four.)
    cfg = DenseConfig(layers=1, max_ctx=8192 + 64)
    host = M.host_model(cfg, "bench-shape")
    weights = M.upload(host, cfg, gpu.put)
    prog = DenseProgram(gpu, cfg, weights, batch, gpu.zeros)
    prog.set_rope_table(gpu.put(DenseProgram.rope_table(cfg)))
    rng = np.random.default_rng(8192)
    positions = np.array([8192 - 3 * b for b in range(batch)], dtype=np.uint32)
    tokens = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    kv_shape = (batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim)
    kc_host = rng.normal(size=kv_shape).astype(np.float16)
    vc_host = rng.normal(size=kv_shape).astype(np.float16)
    prog.kc[0].upload(kc_host.view(np.uint16))
    prog.vc[0].upload(vc_host.view(np.uint16))
    prog.write_step(tokens, positions)
    prog.record_step(int(positions.max()) + 1)
    gpu.sync()
    logits = prog.logits.download(np.float32).reshape(batch, cfg.vocab)
    hidden = prog.x.download(np.float32).reshape(batch, cfg.hidden)
    for b in range(batch):
        kc = [np.ascontiguousarray(kc_host[b]).view(np.uint16).copy()]
        vc = [np.ascontiguousarray(vc_host[b]).view(np.uint16).copy()]
        want_logits, want_x = oracle_step(ref, cfg, host, int(tokens[b]), int(positions[b]), kc, vc)
        assert rel_l2(hidden[b], want_x) < 1e-4, (b, rel_l2(hidden[b], want_x))
        assert rel_l2(logits[b], want_logits) < 1e-4, (b, rel_l2(logits[b], want_logits))
        assert rel_err(logits[b], want_logits) < 1e-3   # the hard ceiling: largest error over the largest logit
        assert int(np.argmax(logits[b])) == int(np.argmax(want_logits))


def test_a_wait_for_an_exchange_that_nobody_pushes_runs_out(gpu, launcher):
    # A multiply told to take its input from an exchange slot that no kernel ever pushes: its wait runs out after the
    # limit the host set (50 ms here, 2 s by default), the kernel returns, the next sync reports the error, and the
    # context works again once the peers are configured again. No hang, no fault: a bounded wait expiring.
    from zllm_b200 import abi, synth

    rng = np.random.default_rng(3)
    n, k = 64, 1024
    w = gpu.put(synth.q4_k_weights(rng, n, k))
    x_host = synth.normal_f32(rng, 1, k)
    arena = abi.PeerArena(gpu, 0, 1, 1 << 16, 4)
    gpu.peer_wait_limit(50)
    x, out = arena.alloc(k * 4), arena.alloc(n * 4)
    x.upload(x_host)
    launcher.matvec("q4_k", x, w, out, n, k, wait=2)
    with pytest.raises(abi.ZcuError) as e:
        gpu.sync()
    assert e.value.name == "GpuError" and "did not arrive" in e.value.message
    # configured again (fresh counts and abort word): a plain multiply and an exchanged pair both work
    arena = abi.PeerArena(gpu, 0, 1, 1 << 16, 4)
    gpu.peer_wait_limit(0)
    x, mid, out = arena.alloc(k * 4), arena.alloc(k * 4), arena.alloc(n * 4)
    x.upload(x_host)
    w2 = gpu.put(synth.q4_k_weights(rng, k, k))
    launcher.matvec("q4_k", x, w2, mid, k, k, push=1)
    launcher.matvec("q4_k", mid, w, out, n, k, wait=1)
    gpu.sync()
    plain_mid, plain_out = gpu.zeros(k * 4), gpu.zeros(n * 4)
    launcher.matvec("q4_k", gpu.put(x_host), w2, plain_mid, k, k)
    launcher.matvec("q4_k", plain_mid, w, plain_out, n, k)
    gpu.sync()
    assert np.array_equal(out.download(np.uint32), plain_out.download(np.uint32))

