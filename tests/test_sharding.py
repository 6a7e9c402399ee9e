"""CPU tier for the multi-GPU path: the plan's sharding arithmetic (which rows, heads and output columns a rank
owns) and the all-gather plumbing, run as two `gloo` ranks. Each rank computes ITS shard of one decode layer
with the CPU oracle in the order the sharded program launches its kernels, gathers where the program gathers,
and the result must equal the unsharded oracle layer."""
import os
import tempfile

import numpy as np
import pytest

from zllm_b200 import kernels as K
from zllm_b200 import model as M
from zllm_b200.plan import DenseConfig, Shard, layer_weight_shapes, shard_rows, slice_full_weights

CFG = DenseConfig(layers=1, hidden=512, heads=8, kv_heads=4, head_dim=64, ff=1024, vocab=1024, max_ctx=64)


def test_shard_shapes_cover_the_model_exactly():
    for world in (1, 2, 4):
        rows = {"wqkv": 0, "wo": 0, "wgu": 0, "wdown": 0}
        for r in range(world):
            for name, (n, k) in layer_weight_shapes(CFG, Shard(r, world)).items():
                rows[name] += n
        assert rows == {"wqkv": CFG.q_dim + 2 * CFG.kv_dim, "wo": CFG.hidden, "wgu": 2 * CFG.ff, "wdown": CFG.hidden}
    assert shard_rows(12, 2, 4) == (6, 9)
    with pytest.raises(AssertionError):
        shard_rows(10, 0, 4)


def test_slices_partition_every_stacked_matrix():
    # Tag each row of the full matrices with its index; the ranks' slices must hold every row exactly once,
    # and stacked parts must stay together (a rank's query heads with its KV heads, gate rows with up rows).
    world = 4
    full = {"wqkv": np.arange(CFG.q_dim + 2 * CFG.kv_dim)[:, None], "wgu": np.arange(2 * CFG.ff)[:, None],
            "wo": np.arange(CFG.hidden)[:, None], "wdown": np.arange(CFG.hidden)[:, None], "head": np.arange(CFG.vocab)[:, None]}
    for name, rows in full.items():
        got = np.concatenate([slice_full_weights(CFG, Shard(r, world), name, rows) for r in range(world)]).ravel()
        assert sorted(got.tolist()) == list(range(rows.shape[0])), name
    sh = Shard(1, world)
    qkv = slice_full_weights(CFG, sh, "wqkv", full["wqkv"]).ravel()
    hd, lh, lg = CFG.head_dim, CFG.heads // world, CFG.kv_heads // world
    assert qkv[0] == 1 * lh * hd and qkv[lh * hd] == CFG.q_dim + 1 * lg * hd
    assert qkv[(lh + lg) * hd] == CFG.q_dim + CFG.kv_dim + 1 * lg * hd
    gu = slice_full_weights(CFG, sh, "wgu", full["wgu"]).ravel()
    lff = CFG.ff // world
    assert gu[0] == lff and gu[lff] == CFG.ff + lff  # up row j sits `half` = lff rows after gate row j


def _rank_main(rank: int, world: int, port: int, out_path: str):
    import torch
    import torch.distributed as dist

    from oracle import ref

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, sh = CFG, Shard(rank, world)
    e, hd = cfg.hidden, cfg.head_dim
    host = M.host_model(cfg, "shard-test")
    lw = host["layers"][0]
    rng = np.random.default_rng(3)
    pos = 40
    x = rng.normal(size=e).astype(np.float32)
    kc = rng.normal(size=(cfg.max_ctx, cfg.kv_heads, hd)).astype(np.float16)
    vc = rng.normal(size=(cfg.max_ctx, cfg.kv_heads, hd)).astype(np.float16)

    def gather(local: np.ndarray) -> np.ndarray:
        parts = [torch.empty(local.size, dtype=torch.float32) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(local, dtype=np.float32)))
        return torch.cat(parts).numpy()

    shapes = layer_weight_shapes(cfg, sh)
    mats = {name: ref.Matrix(ref.Q4_K, slice_full_weights(cfg, sh, name, lw[name]), *shapes[name])
            for name in ("wqkv", "wo", "wgu", "wdown")}
    h0, h1 = sh.heads(cfg)
    g0, g1 = sh.kv_heads(cfg)
    lh, lg = h1 - h0, g1 - g0
    e0, e1 = shard_rows(e, rank, world)
    lff = cfg.ff // world
    # 1. qkv of this rank's heads, 2. rope + cache append (its KV heads), 3-4. attention
    h = ref.rms_norm(x, lw["attn_norm"], cfg.eps)
    qkv = ref.matmul(h, mats["wqkv"])[0]
    q = np.stack([ref.rope_normal(qkv[i * hd:(i + 1) * hd], pos, hd, cfg.rope_base) for i in range(lh)])
    kc_l = np.ascontiguousarray(kc[:, g0:g1]).view(np.uint16).copy()
    vc_l = np.ascontiguousarray(vc[:, g0:g1]).view(np.uint16).copy()
    for i in range(lg):
        k_i = ref.rope_normal(qkv[(lh + i) * hd:(lh + i + 1) * hd], pos, hd, cfg.rope_base)
        kc_l[pos, i] = ref.to_f16_bits(k_i)
        vc_l[pos, i] = ref.to_f16_bits(qkv[(lh + lg + i) * hd:(lh + lg + i + 1) * hd])
    att_local = ref.attend_decode(q, kc_l, vc_l, pos + 1, lh, lg, hd, K.attention_scale(hd))
    att = gather(att_local.ravel())                                    # gather 1: att
    # 5. Wo rows of this rank, accumulated into its slice of x
    x_new = gather(x[e0:e1] + ref.matmul(att, mats["wo"])[0])          # gather 2: x
    # 6. gate|up rows of this rank with SwiGLU
    h = ref.rms_norm(x_new, lw["ffn_norm"], cfg.eps)
    gu = ref.matmul(h, mats["wgu"])[0]
    lib = ref.lib()
    act_local = np.array([lib.ref_silu(float(a)) for a in gu[:lff]], dtype=np.float32) * gu[lff:]
    act = gather(act_local)                                            # gather 3: act
    # 7. Wdown rows of this rank
    x_out = gather(x_new[e0:e1] + ref.matmul(act, mats["wdown"])[0])   # gather 4: x
    if rank == 0:
        np.save(out_path, x_out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_layer(ref):
    import torch.multiprocessing as mp

    cfg = CFG
    e, hd = cfg.hidden, cfg.head_dim
    with tempfile.TemporaryDirectory() as tmp:
        out_path = os.path.join(tmp, "x.npy")
        port = 29600 + os.getpid() % 300
        mp.spawn(_rank_main, args=(2, port, out_path), nprocs=2, join=True)
        got = np.load(out_path)
    host = M.host_model(cfg, "shard-test")
    lw = host["layers"][0]
    rng = np.random.default_rng(3)
    pos = 40
    x = rng.normal(size=e).astype(np.float32)
    kc = rng.normal(size=(cfg.max_ctx, cfg.kv_heads, hd)).astype(np.float16).view(np.uint16)
    vc = rng.normal(size=(cfg.max_ctx, cfg.kv_heads, hd)).astype(np.float16).view(np.uint16)
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
    want = ref.dense_decode_layer(layer, x, kc.copy(), vc.copy(), pos, cfg.heads, cfg.kv_heads, hd, cfg.ff, cfg.eps,
                                  cfg.rope_base, K.attention_scale(hd))
    # every output row, head and column is computed by exactly one rank with the same arithmetic: same bits
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_exchange_slots_chain_through_the_sharded_launch_list():
    # The sharded plan on a dry-run context (no device): every multiply that reads a gathered vector waits for the
    # exchange that the vector's producer pushes, slots are used once per step, and the list ends with the wait
    # that hands the logits to the host.
    import ctypes as C

    from zllm_b200 import abi
    from zllm_b200.plan import DenseProgram

    ctx = abi.Context(dry_run=True)

    class FakeArena:
        def alloc(self, n):
            return ctx.alloc(n)

    cfg = DenseConfig(layers=3, hidden=512, heads=8, kv_heads=4, head_dim=64, ff=1024, vocab=1024, max_ctx=64)
    weights = {"embed": ctx.alloc(256), "head": ctx.alloc(256), "out_norm": ctx.alloc(256),
               "layers": [{k: ctx.alloc(256) for k in ("wqkv", "wo", "wgu", "wdown", "attn_norm", "ffn_norm")} for _ in range(cfg.layers)]}
    prog = DenseProgram(ctx, cfg, weights, 1, ctx.alloc, Shard(1, 2), arena=FakeArena())
    per_layer = 5   # Q|K|V with rope_append, attn_split, the output projection with attn_combine as its first phase, gate|up, down
    prog.set_rope_table(ctx.alloc(256))
    seen = []
    real = prog.L.launch

    def spy(kernel, params, args, groups, variant=0):
        raw = bytes(params)
        ext = K.PeerExt.from_buffer_copy(raw[-16:]) if len(raw) >= 16 else None
        seen.append((kernel, (ext.wait_slot, ext.push_slot) if ext is not None and ext.magic == K.PEER_MAGIC else None))
        real(kernel, params, args, groups, variant)

    prog.L.launch = spy
    before = ctx.launch_count()
    prog.record_step(17)
    assert ctx.launch_count() - before == len(seen) == 2 + per_layer * cfg.layers + 2 == prog.launches_per_step
    none = K.PEER_NONE
    exts = [e for _, e in seen]
    assert exts[0] is None                                    # embed: every rank decodes the row itself
    for il in range(cfg.layers):
        ops = exts[1 + per_layer * il: 1 + per_layer * (il + 1)]
        qkv, (wo, gu, down) = ops[0], ops[-3:]
        assert qkv == (None if il == 0 else (4 * il - 1, none))  # the residual stream of the layer before
        assert ops[1] is None                                    # attn_split
        # the output projection merges the partials, pushes the heads' columns under the slot it waits for, and pushes x
        assert wo == (4 * il, 4 * il + 1) and gu == (4 * il + 1, 4 * il + 2) and down == (4 * il + 2, 4 * il + 3)
    assert exts[-3] == (4 * cfg.layers - 1, 4 * cfg.layers)       # the head
    assert seen[-2] == (K.EXT_PEER_WAIT, (4 * cfg.layers, none))  # the host's wait for the logits
    assert seen[-1] == (K.EXT_PEER_NEXT, (none, none))            # the run ends: the next one tags its exchanges anew
    pushed = [e[1] for e in exts if e is not None and e[1] != none]
    assert sorted(pushed + [4 * il for il in range(cfg.layers)]) == list(range(DenseProgram.arena_slots(cfg)))
    # without the fusion attn_combine is its own launch and pushes the heads' columns itself
    seen.clear()
    prog.fuse_combine = False
    prog.record_step(17)
    assert len(seen) == 2 + 6 * cfg.layers + 2 and [e for _, e in seen][3] == (none, 0)
    assert len(bytes(K.with_peer(K.Matvec(1, 2, 3, 4, 0.0, 0, 0, 0), wait=3))) == C.sizeof(K.Matvec) + 16
    ctx.close()


@pytest.mark.parametrize("batch,sharded", [(1, False), (4, False), (5, False), (8, True), (64, False), (65, False)])
def test_batched_family_is_chosen_for_more_than_four_sequences(batch, sharded):
    # The plan on a dry-run context: steps of 5..64 sequences take the batched tcgen05 family for every Q4_K multiply
    # (also inside a tensor-parallel exchange, where its waits and pushes ride on the same dispatches); the Q8_0 head
    # and smaller or larger steps keep the default family. rope_append is fused only at 1, 2 or 4 sequences.
    from zllm_b200 import abi
    from zllm_b200.plan import DenseProgram

    ctx = abi.Context(dry_run=True)

    class FakeArena:
        def alloc(self, n):
            return ctx.alloc(n)

    cfg = DenseConfig(layers=2, hidden=512, heads=8, kv_heads=4, head_dim=64, ff=1024, vocab=1024, max_ctx=64)
    weights = {"embed": ctx.alloc(256), "head": ctx.alloc(256), "out_norm": ctx.alloc(256),
               "layers": [{k: ctx.alloc(256) for k in ("wqkv", "wo", "wgu", "wdown", "attn_norm", "ffn_norm")} for _ in range(cfg.layers)]}
    prog = DenseProgram(ctx, cfg, weights, batch, ctx.alloc, Shard(1, 2) if sharded else None, arena=FakeArena() if sharded else None)
    prog.set_rope_table(ctx.alloc(256))
    seen = []
    real = prog.L.launch

    def spy(kernel, params, args, groups, variant=0):
        seen.append((kernel, variant, groups))
        real(kernel, params, args, groups, variant)

    prog.L.launch = spy
    prog.record_step(17)
    want = 4 < batch <= K.MATVEC_BATCHED_MAX_TOKENS
    assert prog.batched == want
    q4 = [(v, g) for k, v, g in seen if k == K.MATVEC_KERNEL["q4_k"]]
    assert len(q4) == 4 * cfg.layers and all(g[1] == batch for _, g in q4)
    assert all(v == (K.MATVEC_BATCHED if want else 0) for v, _ in q4)
    head = [(v, g) for k, v, g in seen if k == K.MATVEC_KERNEL["q8_0"]]
    assert head == [(0, head[0][1])]
    rope_launches = sum(1 for k, _, _ in seen if k == K.ROPE_APPEND)
    assert rope_launches == (0 if batch in (1, 2, 4) else cfg.layers)
    ctx.close()


# ---- the hybrid model: DeltaNet layers sharded by value head
from zllm_b200.plan import HybridConfig, delta_shard, slice_delta_weights  # noqa: E402

HCFG = HybridConfig(layers=4, hidden=512, heads=8, kv_heads=2, head_dim=64, ff=1024, vocab=1024, max_ctx=64,
                    gdn_head_dim=64, gdn_k_heads=2, gdn_v_heads=4, conv_kernel=4, attention_every=4)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_value_head_shards_keep_the_key_heads_they_use(world):
    cfg = HCFG
    d, hk, hv = cfg.gdn_head_dim, cfg.gdn_k_heads, cfg.gdn_v_heads
    conv_dim = 2 * hk * d + hv * d
    rows = conv_dim + hv * d + 2 * hv
    full = np.arange(rows, dtype=np.int64)[:, None]          # each row holds its own index
    seen_v = []
    for rank in range(world):
        v0, lv, k0, lk = delta_shard(cfg, Shard(rank, world))
        # local value head j uses local key head j mod lk: the global head it maps to is the one the full model uses
        assert all((k0 + j % lk) == (v0 + j) % hk for j in range(lv))
        got = slice_delta_weights(cfg, Shard(rank, world), "wproj", full).ravel()
        q, k, v = got[:lk * d], got[lk * d:2 * lk * d], got[2 * lk * d:2 * lk * d + lv * d]
        assert q[0] == k0 * d and k[0] == hk * d + k0 * d and v[0] == 2 * hk * d + v0 * d
        z = got[2 * lk * d + lv * d:2 * lk * d + 2 * lv * d]
        assert z[0] == conv_dim + v0 * d and got[-2 * lv] == conv_dim + hv * d + v0 and got[-lv] == conv_dim + hv * d + hv + v0
        assert slice_delta_weights(cfg, Shard(rank, world), "conv", full[:conv_dim]).shape[0] == 2 * lk * d + lv * d
        seen_v += list(range(v0, v0 + lv))
    assert seen_v == list(range(hv))


def _delta_layer(ref, cfg, lw_mats, lw, x_rows, hk, hv):
    """A DeltaNet mixer over consecutive tokens on the oracle, with `hk` key and `hv` value heads: the columns of o."""
    d, taps = cfg.gdn_head_dim, cfg.conv_kernel
    cd, inner = 2 * hk * d + hv * d, hv * d
    n = x_rows.shape[0]
    h = np.stack([ref.rms_norm(x, lw["attn_norm"], cfg.eps) for x in x_rows])
    proj = ref.matmul(h, lw_mats["wproj"])
    conv = ref.conv_norm(proj[:, :cd].copy(), lw_mats["conv"], n, hk, inner, d, taps, cfg.eps)
    beta = (1 / (1 + np.exp(-proj[:, cd + inner:cd + inner + hv].astype(np.float64)))).astype(np.float32)
    g = (np.log1p(np.exp(proj[:, cd + inner + hv:].astype(np.float64) + lw_mats["dt_bias"])) * lw_mats["a"]).astype(np.float32)
    _, o = ref.delta_rule(np.zeros((hv, d, d), dtype=np.float32), conv, g, beta, n, hk, hv, d)
    return ref.gated_norm(o, proj[:, cd:cd + inner].copy(), lw["norm"], n, hv, d, cfg.eps)


def _hybrid_rank_main(rank: int, world: int, port: int, out_path: str):
    import torch
    import torch.distributed as dist

    from oracle import ref

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, sh = HCFG, Shard(rank, world)
    e = cfg.hidden
    lw = M.hybrid_host_model(cfg, "hybrid-shard")["layers"][0]
    x_rows = np.random.default_rng(5).normal(size=(3, e)).astype(np.float32)
    _, lv, _, lk = delta_shard(cfg, sh)
    sl = {name: slice_delta_weights(cfg, sh, name, lw[name]) for name in ("wproj", "conv", "dt_bias", "a", "wout")}
    mats = dict(sl, wproj=ref.Matrix(ref.Q4_K, sl["wproj"], sl["wproj"].shape[0], e))
    o_local = _delta_layer(ref, cfg, mats, lw, x_rows, lk, lv)            # [tokens, lv * d]
    parts = [torch.empty(o_local.shape, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(o_local)))
    o = torch.cat(parts, dim=1).numpy()                                    # exchange: head columns
    e0, e1 = shard_rows(e, rank, world)
    x_local = x_rows[:, e0:e1] + ref.matmul(o, ref.Matrix(ref.Q4_K, sl["wout"], e1 - e0, cfg.gdn_inner))
    parts = [torch.empty(x_local.shape, dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(x_local)))
    if rank == 0:
        np.save(out_path, torch.cat(parts, dim=1).numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_deltanet_layer(ref):
    import torch.multiprocessing as mp

    cfg, e = HCFG, HCFG.hidden
    with tempfile.TemporaryDirectory() as tmp:
        out_path = os.path.join(tmp, "x.npy")
        port = 29950 + os.getpid() % 300
        mp.spawn(_hybrid_rank_main, args=(2, port, out_path), nprocs=2, join=True)
        got = np.load(out_path)
    lw = M.hybrid_host_model(cfg, "hybrid-shard")["layers"][0]
    x_rows = np.random.default_rng(5).normal(size=(3, e)).astype(np.float32)
    mats = dict(lw, wproj=ref.Matrix(ref.Q4_K, lw["wproj"], lw["wproj"].shape[0], e))
    o = _delta_layer(ref, cfg, mats, lw, x_rows, cfg.gdn_k_heads, cfg.gdn_v_heads)
    want = x_rows + ref.matmul(o, ref.Matrix(ref.Q4_K, lw["wout"], e, cfg.gdn_inner))
    # every head and every output row is computed by exactly one rank with the same arithmetic: same bits
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_exchange_slots_chain_through_the_sharded_hybrid_launch_list():
    # DeltaNet layers use the same four exchanges per layer as attention layers: gated_norm pushes the rank's head
    # columns where attn_combine would, the output projection waits for them.
    from zllm_b200 import abi
    from zllm_b200.plan import HybridProgram

    ctx = abi.Context(dry_run=True)

    class FakeArena:
        def alloc(self, n):
            return ctx.alloc(n)

    cfg = HCFG
    names = {True: ("wqkv", "wo"), False: ("wproj", "conv", "dt_bias", "a", "norm", "wout")}
    weights = {"embed": ctx.alloc(256), "head": ctx.alloc(256), "out_norm": ctx.alloc(256),
               "layers": [{k: ctx.alloc(256) for k in names[cfg.is_attention(il)] + ("wgu", "wdown", "attn_norm", "ffn_norm")}
                          for il in range(cfg.layers)]}
    prog = HybridProgram(ctx, cfg, weights, 1, ctx.alloc, Shard(1, 2), arena=FakeArena())
    prog.set_rope_table(ctx.alloc(256))
    assert (prog.lvh, prog.lkh, prog.v0, prog.k0) == (2, 2, 2, 0)
    assert [c is not None for c in prog.kc] == [False, False, False, True]
    seen = []
    real = prog.L.launch

    def spy(kernel, params, args, groups, variant=0):
        raw = bytes(params)
        ext = K.PeerExt.from_buffer_copy(raw[-16:]) if len(raw) >= 16 else None
        seen.append((kernel, (ext.wait_slot, ext.push_slot) if ext is not None and ext.magic == K.PEER_MAGIC else None))
        real(kernel, params, args, groups, variant)

    prog.L.launch = spy
    prog.record_step(9)
    none = K.PEER_NONE
    assert len(seen) == prog.launches_per_step                  # the host's wait for the logits included
    i = 1
    for il in range(cfg.layers):
        n = 5 if cfg.is_attention(il) else 7   # (an attention layer's output projection merges the attention's partials itself)
        ops = seen[i:i + n]
        i += n
        assert ops[0][1] == (None if il == 0 else (4 * il - 1, none))
        if not cfg.is_attention(il):
            assert [k for k, _ in ops[1:4]] == [K.DELTA_PREP, K.DELTA_RULE, K.GATED_NORM]
            assert ops[1][1] is None and ops[2][1] is None and ops[3][1] == (none, 4 * il)
        assert [e for _, e in ops[-3:]] == [(4 * il, 4 * il + 1), (4 * il + 1, 4 * il + 2), (4 * il + 2, 4 * il + 3)]
    pushed = [e[1] for _, e in seen if e is not None and e[1] != none]
    pushed += [4 * il for il in range(cfg.layers) if cfg.is_attention(il)]   # pushed by the output projection's first phase
    assert sorted(pushed) == list(range(HybridProgram.arena_slots(cfg)))
    ctx.close()


def test_pick_trial_keeps_the_default_unless_a_trial_beats_it_by_the_margin():
    from zllm_b200.plan import DenseProgram

    pick = DenseProgram.pick_trial
    assert pick([1.000, 0.999, 0.998, 1.2], 0.003) == 0          # within the margin: the default stays
    assert pick([1.000, 0.990, 0.985, 1.2], 0.003) == 2          # the fastest trial beyond the margin
    assert pick([1.000, 1.1, 1.2, 1.3], 0.003) == 0
    assert pick([1.000], 0.003) == 0
    # the ranks decide by the times `agree` returns (here: another rank was slow in trial 2)
    assert pick([1.000, 0.990, 0.985, 1.2], 0.003, agree=lambda t: [max(a, b) for a, b in zip(t, [1.0, 0.991, 1.05, 1.0])]) == 1


def _agree_main(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist

    from zllm_b200.plan import DenseProgram

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def agree(times):
        t = torch.tensor(times, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    # each rank alone would keep another trial (rank 0: trial 1, rank 1: trial 2); together they keep trial 3, the one
    # whose slowest rank is fastest
    mine = [[1.0, 0.90, 1.10, 0.95], [1.0, 1.10, 0.90, 0.94]][rank]
    alone = DenseProgram.pick_trial(mine, 0.003)
    together = DenseProgram.pick_trial(mine, 0.003, agree)
    with open(os.path.join(out_dir, f"pick{rank}.txt"), "w") as f:
        f.write(f"{alone} {together}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_keep_the_same_trial():
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as tmp:
        port = 29900 + os.getpid() % 90
        mp.spawn(_agree_main, args=(2, port, tmp), nprocs=2, join=True)
        picks = [open(os.path.join(tmp, f"pick{r}.txt")).read().split() for r in range(2)]
    assert picks == [["1", "3"], ["2", "3"]]
