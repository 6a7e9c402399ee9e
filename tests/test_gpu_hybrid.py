"""A hybrid model's decode step (Gated DeltaNet layers with an attention layer every few, src/graph/qwen35.zig:21-56,
src/plan/qwen35.zig:556-599) against the CPU oracle composed layer by layer: consecutive steps from an empty
sequence, so the recurrent states, the conv histories and the KV cache are all carried by the program."""
import numpy as np
import pytest

from tests.util import rel_l2
from zllm_b200 import kernels as K
from zllm_b200 import model as M
from zllm_b200.plan import HybridConfig, HybridProgram

pytestmark = pytest.mark.gpu

CFG = HybridConfig(layers=4, hidden=512, heads=8, kv_heads=2, head_dim=64, ff=1024, vocab=1536, max_ctx=192,
                   gdn_head_dim=64, gdn_k_heads=2, gdn_v_heads=4, conv_kernel=4, attention_every=4)


class OracleHybrid:
    """One sequence on the oracle: per DeltaNet layer the raw conv inputs seen so far and the state."""

    def __init__(self, ref, cfg, host):
        self.ref, self.cfg, self.host = ref, cfg, host
        d, hv = cfg.gdn_head_dim, cfg.gdn_v_heads
        self.conv_dim = 2 * cfg.gdn_k_heads * d + hv * d
        self.seen = {il: np.zeros((0, self.conv_dim), dtype=np.float32) for il in range(cfg.layers)}
        self.state = {il: np.zeros((hv, d, d), dtype=np.float32) for il in range(cfg.layers)}
        self.kc = [np.zeros((cfg.max_ctx, cfg.kv_heads, cfg.head_dim), dtype=np.uint16) for _ in range(cfg.layers)]
        self.vc = [np.zeros((cfg.max_ctx, cfg.kv_heads, cfg.head_dim), dtype=np.uint16) for _ in range(cfg.layers)]

    def ffn(self, lw, x):
        ref, cfg, e = self.ref, self.cfg, self.cfg.hidden
        h = ref.rms_norm(x, lw["ffn_norm"], cfg.eps)
        gate = ref.matmul(h, ref.Matrix(ref.Q4_K, lw["wgu"][:cfg.ff], cfg.ff, e))[0]
        up = ref.matmul(h, ref.Matrix(ref.Q4_K, lw["wgu"][cfg.ff:], cfg.ff, e))[0]
        act = (gate / (1 + np.exp(-gate.astype(np.float64)))).astype(np.float32) * up
        return x + ref.matmul(act, ref.Matrix(ref.Q4_K, lw["wdown"], e, cfg.ff))[0]

    def delta_layer(self, il, lw, x):
        ref, cfg, e = self.ref, self.cfg, self.cfg.hidden
        d, hk, hv, taps = cfg.gdn_head_dim, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.conv_kernel
        inner, cd = hv * d, self.conv_dim
        h = ref.rms_norm(x, lw["attn_norm"], cfg.eps)
        proj = ref.matmul(h, ref.Matrix(ref.Q4_K, lw["wproj"], lw["wproj"].shape[0], e))[0]
        self.seen[il] = np.concatenate([self.seen[il], proj[None, :cd]])
        n = self.seen[il].shape[0]
        conv = ref.conv_norm(self.seen[il].copy(), lw["conv"], n, hk, inner, d, taps, cfg.eps)[n - 1:]
        beta = 1 / (1 + np.exp(-proj[cd + inner:cd + inner + hv].astype(np.float64)))
        xa = proj[cd + inner + hv:cd + inner + 2 * hv].astype(np.float64) + lw["dt_bias"]
        g = np.log1p(np.exp(xa)) * lw["a"]
        self.state[il], o = ref.delta_rule(self.state[il], conv, g.astype(np.float32)[None], beta.astype(np.float32)[None], 1,
                                           hk, hv, d, mode=ref.F64)
        o = ref.gated_norm(o, proj[None, cd:cd + inner].copy(), lw["norm"], 1, hv, d, cfg.eps)[0]
        return x + ref.matmul(o, ref.Matrix(ref.Q4_K, lw["wout"], e, inner))[0]

    def step(self, token, pos):
        ref, cfg, e = self.ref, self.cfg, self.cfg.hidden
        x = ref.dequantize(ref.Q4_K, self.host["embed"][token], e)
        for il, lw in enumerate(self.host["layers"]):
            if cfg.is_attention(il):
                rows = lw["wqkv"]
                layer = {"attn_norm": lw["attn_norm"], "ffn_norm": lw["ffn_norm"],
                         "wq": ref.Matrix(ref.Q4_K, rows[:cfg.q_dim], cfg.q_dim, e),
                         "wk": ref.Matrix(ref.Q4_K, rows[cfg.q_dim:cfg.q_dim + cfg.kv_dim], cfg.kv_dim, e),
                         "wv": ref.Matrix(ref.Q4_K, rows[cfg.q_dim + cfg.kv_dim:], cfg.kv_dim, e),
                         "wo": ref.Matrix(ref.Q4_K, lw["wo"], e, cfg.q_dim),
                         "gate": ref.Matrix(ref.Q4_K, lw["wgu"][:cfg.ff], cfg.ff, e),
                         "up": ref.Matrix(ref.Q4_K, lw["wgu"][cfg.ff:], cfg.ff, e),
                         "down": ref.Matrix(ref.Q4_K, lw["wdown"], e, cfg.ff)}
                x = ref.dense_decode_layer(layer, x, self.kc[il], self.vc[il], pos, cfg.heads, cfg.kv_heads, cfg.head_dim,
                                           cfg.ff, cfg.eps, cfg.rope_base, K.attention_scale(cfg.head_dim))
            else:
                x = self.ffn(lw, self.delta_layer(il, lw, x))
        return self.ref.dense_head(x, self.host["out_norm"], ref.Matrix(ref.Q8_0, self.host["head"], cfg.vocab, e), cfg.eps), x


def fresh(gpu, cfg, weights, **kw):
    prog = HybridProgram(gpu, cfg, weights, 1, gpu.zeros, **kw)
    prog.set_rope_table(gpu.put(HybridProgram.rope_table(cfg)))
    return prog


def test_hybrid_steps_match_the_oracle(ref, gpu):
    cfg = CFG
    host = M.hybrid_host_model(cfg, "hybrid-tiny")
    prog = fresh(gpu, cfg, M.upload_hybrid(host, cfg, gpu.put))
    oracle = OracleHybrid(ref, cfg, host)
    for pos, token in enumerate([11, 700, 3, 1500, 42, 42]):
        prog.write_step(np.array([token], dtype=np.uint32), np.array([pos], dtype=np.uint32))
        prog.record_step(pos + 1)
        gpu.sync()
        want_logits, want_x = oracle.step(token, pos)
        got = prog.logits.download(np.float32)
        assert rel_l2(prog.x.download(np.float32), want_x) < 1e-4, (pos, rel_l2(prog.x.download(np.float32), want_x))
        assert rel_l2(got, want_logits) < 1e-4, (pos, rel_l2(got, want_logits))
        assert int(np.argmax(got)) == int(np.argmax(want_logits))
    # embedding; a DeltaNet layer = projection, prep, rule, norm, output projection + 2 FFN; the attention layer; head
    assert prog.launches_per_step == 1 + 3 * 7 + (7 - prog.fuse_rope) + 1
    for il in (0, 2):
        assert rel_l2(prog.state[il].download(np.float32), oracle.state[il].ravel()) < 1e-4
        # the history holds the last taps-1 raw conv inputs, oldest first
        assert rel_l2(prog.hist[il].download(np.float32), oracle.seen[il][-(cfg.conv_kernel - 1):].ravel()) < 1e-4


def test_hybrid_peer_exchange_with_one_rank_equals_the_plain_step(gpu):
    # gated_norm publishes its heads like attn_combine does; a world of one goes through the same pushes and waits.
    from zllm_b200 import abi

    cfg = CFG
    host = M.hybrid_host_model(cfg, "hybrid-tiny")
    weights = M.upload_hybrid(host, cfg, gpu.put)
    arena = abi.PeerArena(gpu, 0, 1, HybridProgram.arena_bytes(cfg, 1), HybridProgram.arena_slots(cfg))
    plain, peer = fresh(gpu, cfg, weights), fresh(gpu, cfg, weights, arena=arena)
    graph = None
    for pos, token in enumerate([9, 1000, 77, 5]):
        for p in (plain, peer):
            p.write_step(np.array([token], dtype=np.uint32), np.array([pos], dtype=np.uint32))
        plain.record_step(cfg.max_ctx)
        if graph is None:
            gpu.sync()
            gpu.capture_begin()
            peer.record_step(cfg.max_ctx)
            graph = gpu.capture_end()
        gpu.graph_launch(graph)
        gpu.sync()
        for name in ("logits", "x", "o", "act"):
            assert np.array_equal(getattr(plain, name).download(np.uint32), getattr(peer, name).download(np.uint32)), (name, pos)
