"""Tensor parallelism on real devices: a decode step sharded over two GPUs (rows, heads and KV heads per
rank, NCCL all-gather of output slices) gives the logits of the same step on one GPU, bit for bit: every
output row, head and column is computed by exactly one rank with the same arithmetic. Needs two GPUs."""
import os
import tempfile
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rank(rank: int, world: int, port: int, out_dir: str):
    import torch
    import torch.distributed as dist

    from zllm_b200 import abi
    from zllm_b200 import model as M
    from zllm_b200.plan import DenseConfig, DenseProgram, Shard
    from zllm_b200.torch_util import TorchBuf, nccl_gather

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    cfg = DenseConfig(layers=2, hidden=512, heads=8, kv_heads=2, head_dim=64, ff=1024, vocab=1536, max_ctx=320)
    host = M.host_model(cfg, "tp-test")
    rng = np.random.default_rng(17)
    batch = 2
    positions = np.array([100, 37], dtype=np.uint32)
    tokens = rng.integers(0, cfg.vocab, size=batch).astype(np.uint32)
    kv_shape = (batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim)
    kc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    vc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    results = {}
    for w in ((1, world) if rank == 0 else (world,)):
        sh = Shard(rank if w > 1 else 0, w)
        stream = torch.cuda.Stream(dev)
        ctx = abi.Context(rank, stream=stream.cuda_stream)
        keep = []

        def alloc(n):
            b = TorchBuf(torch, dev, n)
            keep.append(b)
            return b

        def put(a):
            a = np.ascontiguousarray(a)
            return alloc(a.nbytes).upload(a)

        weights = M.upload(host, cfg, put, sh)
        prog = DenseProgram(ctx, cfg, weights, batch, alloc, sh, gather=nccl_gather(dist, rank, w) if w > 1 else None)
        prog.set_rope_table(put(DenseProgram.rope_table(cfg)))
        g0, g1 = sh.kv_heads(cfg)
        for il in range(cfg.layers):
            prog.kc[il].upload(np.ascontiguousarray(kc_host[il][:, :, g0:g1]).view(np.uint16))
            prog.vc[il].upload(np.ascontiguousarray(vc_host[il][:, :, g0:g1]).view(np.uint16))
        prog.write_step(tokens, positions)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            prog.record_step(int(positions.max()) + 1)
        stream.synchronize()
        results[w] = prog.logits.download(np.float32).reshape(batch, cfg.vocab).copy()
        ctx.close()
    if rank == 0:
        np.save(os.path.join(out_dir, "one.npy"), results[1])
        np.save(os.path.join(out_dir, "two.npy"), results[world])
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)  # no NCCL teardown: see bench.py


def _rank_peer(rank: int, world: int, port: int, out_dir: str):
    """The same comparison with the library's own exchange: arenas mapped over CUDA IPC, outputs pushed by the
    kernels' epilogues, counters instead of collectives. torch.distributed (gloo) only carries the IPC handles."""
    import torch.distributed as dist

    from zllm_b200 import abi
    from zllm_b200 import model as M
    from zllm_b200.plan import DenseConfig, DenseProgram, Shard

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = DenseConfig(layers=2, hidden=512, heads=8, kv_heads=2, head_dim=64, ff=1024, vocab=1536, max_ctx=320)
    host = M.host_model(cfg, "tp-test")
    rng = np.random.default_rng(17)
    # six sequences: more than one pass of the multiplies takes (four tokens), so one dispatch pushes its slices in
    # two launches under one exchange tag
    batch = 6
    kv_shape = (batch, cfg.max_ctx, cfg.kv_heads, cfg.head_dim)
    kc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    vc_host = [rng.normal(size=kv_shape).astype(np.float16) for _ in range(cfg.layers)]
    first = np.array([100, 37, 5, 200, 64, 11])
    steps = [(rng.integers(0, cfg.vocab, size=batch).astype(np.uint32), (first + i).astype(np.uint32)) for i in range(3)]
    ctx = abi.Context(rank)

    def exchange(handle: bytes):
        got = [None] * world
        dist.all_gather_object(got, handle)
        return got

    def build(sh, arena, batched=False):
        weights = M.upload(host, cfg, ctx.put, sh)
        # (batched=False: the one-GPU program too takes the mma.sync family, whose bits the sharded one must give)
        prog = DenseProgram(ctx, cfg, weights, batch, ctx.zeros, sh, arena=arena, batched=batched)
        prog.set_rope_table(ctx.put(DenseProgram.rope_table(cfg)))
        g0, g1 = sh.kv_heads(cfg)
        for il in range(cfg.layers):
            prog.kc[il].upload(np.ascontiguousarray(kc_host[il][:, :, g0:g1]).view(np.uint16))
            prog.vc[il].upload(np.ascontiguousarray(vc_host[il][:, :, g0:g1]).view(np.uint16))
        return prog

    arena = abi.PeerArena(ctx, rank, world, DenseProgram.arena_bytes(cfg, batch), DenseProgram.arena_slots(cfg), exchange)
    sharded = build(Shard(rank, world), arena)
    whole = build(Shard(0, 1), None) if rank == 0 else None
    dist.barrier()
    graph, got, want = None, [], []
    for tokens, positions in steps:
        sharded.write_step(tokens, positions)
        if graph is None:
            ctx.sync()
            ctx.capture_begin()
            sharded.record_step(cfg.max_ctx)
            graph = ctx.capture_end()
        ctx.graph_launch(graph)
        ctx.sync()
        got.append(sharded.logits.download(np.float32).reshape(batch, cfg.vocab).copy())
        if whole is not None:
            whole.write_step(tokens, positions)
            whole.record_step(cfg.max_ctx)
            ctx.sync()
            want.append(whole.logits.download(np.float32).reshape(batch, cfg.vocab).copy())
        dist.barrier()  # a rank leaves a step only when every rank has read its logits
    # the same steps with the batched tcgen05 family in the exchange (its column kernel waits on the slots, its
    # reduction pushes): a second arena, since the first program owns the first one's buffers
    arena2 = abi.PeerArena(ctx, rank, world, DenseProgram.arena_bytes(cfg, batch), DenseProgram.arena_slots(cfg), exchange)
    sharded2 = build(Shard(rank, world), arena2, batched=True)
    assert sharded2.batched
    dist.barrier()
    got2 = []
    for tokens, positions in steps:
        sharded2.write_step(tokens, positions)
        sharded2.record_step(cfg.max_ctx)
        ctx.sync()
        got2.append(sharded2.logits.download(np.float32).reshape(batch, cfg.vocab).copy())
        dist.barrier()
    np.save(os.path.join(out_dir, f"peer_batched{rank}.npy"), np.stack(got2))
    if rank == 0:
        np.save(os.path.join(out_dir, "one.npy"), np.stack(want))
    np.save(os.path.join(out_dir, f"peer{rank}.npy"), np.stack(got))
    dist.barrier()
    os._exit(0)


def _spawn(fn, tmp):
    import torch.multiprocessing as mp

    port = 29700 + os.getpid() % 200
    ctx = mp.spawn(fn, args=(2, port, tmp), nprocs=2, join=False)
    deadline = time.monotonic() + 240
    while not ctx.join(timeout=5):  # join() returns as soon as one rank ends; True once all have
        if time.monotonic() > deadline:
            for p in ctx.processes:
                p.kill()  # the two PIDs this test started
            pytest.fail("the two ranks did not finish in 240 s")


def test_two_gpus_with_peer_pushes_give_the_single_gpu_logits():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with tempfile.TemporaryDirectory() as tmp:
        _spawn(_rank_peer, tmp)
        one = np.load(os.path.join(tmp, "one.npy"))
        peers = [np.load(os.path.join(tmp, f"peer{r}.npy")) for r in range(2)]
        batched = [np.load(os.path.join(tmp, f"peer_batched{r}.npy")) for r in range(2)]
    assert np.isfinite(one).all() and np.abs(one).max() > 0
    for r in range(2):  # every rank holds the whole logits, and they are the single-GPU bits
        assert np.array_equal(one.view(np.uint32), peers[r].view(np.uint32)), r
    # the batched family sums in another order (k slices, two f16 terms): the same logits within the model-tier bound,
    # and every rank holds the same bits
    assert np.array_equal(batched[0].view(np.uint32), batched[1].view(np.uint32))
    for step in range(one.shape[0]):
        for b in range(one.shape[1]):
            d = batched[0][step, b].astype(np.float64) - one[step, b]
            assert np.linalg.norm(d) / np.linalg.norm(one[step, b]) < 1e-4, (step, b)
            assert int(np.argmax(batched[0][step, b])) == int(np.argmax(one[step, b]))


def test_two_gpus_give_the_single_gpu_logits():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with tempfile.TemporaryDirectory() as tmp:
        port = 29700 + os.getpid() % 200
        ctx = mp.spawn(_rank, args=(2, port, tmp), nprocs=2, join=False)
        deadline = time.monotonic() + 240
        while not ctx.join(timeout=5):  # join() returns as soon as one rank ends; True once all have
            if time.monotonic() > deadline:
                for p in ctx.processes:
                    p.kill()  # the two PIDs this test started
                pytest.fail("the two ranks did not finish in 240 s")
        one, two = np.load(os.path.join(tmp, "one.npy")), np.load(os.path.join(tmp, "two.npy"))
    assert np.isfinite(one).all() and np.abs(one).max() > 0
    assert np.array_equal(one.view(np.uint32), two.view(np.uint32))


def _rank_peer_hybrid(rank: int, world: int, port: int, out_dir: str):
    """A hybrid model (DeltaNet layers sharded by value head, the recurrent states and conv histories per rank)
    over the library's exchange: consecutive steps of one sequence from an empty state against one GPU."""
    import torch.distributed as dist

    from zllm_b200 import abi
    from zllm_b200 import model as M
    from zllm_b200.plan import HybridConfig, HybridProgram, Shard

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = HybridConfig(layers=4, hidden=512, heads=8, kv_heads=2, head_dim=64, ff=1024, vocab=1536, max_ctx=192,
                       gdn_head_dim=64, gdn_k_heads=2, gdn_v_heads=4, conv_kernel=4, attention_every=4)
    host = M.hybrid_host_model(cfg, "tp-hybrid")
    ctx = abi.Context(rank)

    def exchange(handle: bytes):
        got = [None] * world
        dist.all_gather_object(got, handle)
        return got

    def build(sh, arena):
        prog = HybridProgram(ctx, cfg, M.upload_hybrid(host, cfg, ctx.put, sh), 1, ctx.zeros, sh, arena=arena)
        prog.set_rope_table(ctx.put(HybridProgram.rope_table(cfg)))
        return prog

    arena = abi.PeerArena(ctx, rank, world, HybridProgram.arena_bytes(cfg, 1), HybridProgram.arena_slots(cfg), exchange)
    sharded = build(Shard(rank, world), arena)
    whole = build(Shard(0, 1), None) if rank == 0 else None
    dist.barrier()
    graph, got, want = None, [], []
    for pos, token in enumerate([11, 700, 3, 1500, 42]):
        tok, ps = np.array([token], dtype=np.uint32), np.array([pos], dtype=np.uint32)
        sharded.write_step(tok, ps)
        if graph is None:
            ctx.sync()
            ctx.capture_begin()
            sharded.record_step(cfg.max_ctx)
            graph = ctx.capture_end()
        ctx.graph_launch(graph)
        ctx.sync()
        got.append(sharded.logits.download(np.float32).copy())
        if whole is not None:
            whole.write_step(tok, ps)
            whole.record_step(cfg.max_ctx)
            ctx.sync()
            want.append(whole.logits.download(np.float32).copy())
        dist.barrier()
    if rank == 0:
        np.save(os.path.join(out_dir, "one.npy"), np.stack(want))
        v0, lv = sharded.v0, sharded.lvh
        d = cfg.gdn_head_dim
        np.save(os.path.join(out_dir, "state_one.npy"), whole.state[0].download(np.float32).reshape(-1, d, d)[v0:v0 + lv])
    np.save(os.path.join(out_dir, f"state{rank}.npy"), sharded.state[0].download(np.float32))
    np.save(os.path.join(out_dir, f"peer{rank}.npy"), np.stack(got))
    dist.barrier()
    os._exit(0)


def test_two_gpus_hybrid_with_value_heads_sharded_give_the_single_gpu_logits():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with tempfile.TemporaryDirectory() as tmp:
        _spawn(_rank_peer_hybrid, tmp)
        one = np.load(os.path.join(tmp, "one.npy"))
        peers = [np.load(os.path.join(tmp, f"peer{r}.npy")) for r in range(2)]
        state_one, state0 = np.load(os.path.join(tmp, "state_one.npy")), np.load(os.path.join(tmp, "state0.npy"))
    assert np.isfinite(one).all() and np.abs(one).max() > 0
    # a head's recurrence, a row's multiply: each on exactly one rank with the same arithmetic
    assert np.array_equal(state_one.ravel().view(np.uint32), state0.view(np.uint32))
    for r in range(2):
        assert np.array_equal(one.view(np.uint32), peers[r].view(np.uint32)), r
