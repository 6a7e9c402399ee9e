"""Random-init weights of a Llama-shaped dense model in the kernels' layouts (synthetic: there is no
model file here). Host (numpy) generation for test-sized models, so the same bytes can be handed to a
checker; device (torch) generation for benchmark-sized ones."""
from __future__ import annotations

import numpy as np

from . import kernels as K
from . import synth
from .plan import DenseConfig, Shard, layer_weight_shapes, shard_rows, slice_full_weights


def _quant(rng, ttype: str, n: int, k: int) -> np.ndarray:
    """File-layout rows of `ttype` [n, row bytes in the file]."""
    if ttype == "q4_k":
        return synth.q4_k_weights(rng, n, k, 1e-4, 1e-2)
    if ttype == "q8_0":
        return synth.q8_0_weights(rng, n, k, 1e-4, 2e-3)
    raise ValueError(ttype)


def split_q8_0_rows(file_rows: np.ndarray, k: int) -> np.ndarray:
    """Q8_0 file rows -> the split rows the kernels read (what repack_q8_0 produces)."""
    n = file_rows.shape[0]
    blocks = file_rows.reshape(n, k // 32, 34)
    stride = (k + k // 16 + 15) & ~15
    out = np.zeros((n, stride), dtype=np.uint8)
    out[:, :k] = blocks[:, :, 2:].reshape(n, k)
    out[:, k:k + k // 16] = blocks[:, :, :2].reshape(n, k // 16)
    return out


def host_model(cfg: DenseConfig, seed: str = "model"):
    """The full (unsharded) model on the host: file-layout weight bytes, stacked as the plan stacks them."""
    layers = []
    for il in range(cfg.layers):
        r = lambda name: synth.rng_for(seed, f"l{il}.{name}")  # noqa: E731
        layers.append({
            "wqkv": _quant(r("wqkv"), cfg.body_type, cfg.q_dim + 2 * cfg.kv_dim, cfg.hidden),
            "wo": _quant(r("wo"), cfg.body_type, cfg.hidden, cfg.q_dim),
            "wgu": _quant(r("wgu"), cfg.body_type, 2 * cfg.ff, cfg.hidden),
            "wdown": _quant(r("wdown"), cfg.body_type, cfg.hidden, cfg.ff),
            "attn_norm": (1 + 0.1 * r("attn_norm").normal(size=cfg.hidden)).astype(np.float32),
            "ffn_norm": (1 + 0.1 * r("ffn_norm").normal(size=cfg.hidden)).astype(np.float32),
        })
    return {
        "layers": layers,
        "embed": _quant(synth.rng_for(seed, "embed"), cfg.embed_type, cfg.vocab, cfg.hidden),
        "head": _quant(synth.rng_for(seed, "head"), cfg.head_type, cfg.vocab, cfg.hidden),
        "out_norm": (1 + 0.1 * synth.rng_for(seed, "out_norm").normal(size=cfg.hidden)).astype(np.float32),
    }


def upload(host, cfg: DenseConfig, put, shard: Shard | None = None):
    """Device weights of one rank from a host model; `put(ndarray)` uploads and returns a buffer."""
    sh = shard or Shard()

    def layout(ttype, rows, k):
        return split_q8_0_rows(rows, k) if ttype == "q8_0" else rows

    layers = []
    for lw in host["layers"]:
        d = {}
        for name, k in (("wqkv", cfg.hidden), ("wo", cfg.q_dim), ("wgu", cfg.hidden), ("wdown", cfg.ff)):
            d[name] = put(layout(cfg.body_type, slice_full_weights(cfg, sh, name, lw[name]), k))
        d["attn_norm"] = put(lw["attn_norm"])
        d["ffn_norm"] = put(lw["ffn_norm"])
        layers.append(d)
    return {
        "layers": layers,
        "embed": put(layout(cfg.embed_type, host["embed"], cfg.hidden)),
        "head": put(layout(cfg.head_type, slice_full_weights(cfg, sh, "head", host["head"]), cfg.hidden)),
        "out_norm": put(host["out_norm"]),
    }


def device_model(cfg: DenseConfig, torch, dev, shard: Shard | None = None, seed: int = 0):
    """Benchmark-sized random weights generated on the device: random bytes (nibbles uniform 0..15, 6-bit
    scales/mins uniform 0..63, int8 quants uniform) with f16 super-scales uniform in [1e-4, 1e-2] (Q4_K) or
    [1e-4, 2e-3] (Q8_0). Returns ({name: (ptr, nbytes)} in plan layout, the tensors that own the memory)."""
    sh = shard or Shard()
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + 7919 * sh.rank)
    keep = []

    def q4k(n, k):
        nb = k // 256
        w = torch.randint(0, 256, (n, nb, 144), dtype=torch.uint8, device=dev, generator=gen)
        d = (torch.rand((n, nb, 2), device=dev, generator=gen) * (1e-2 - 1e-4) + 1e-4).to(torch.float16)
        w[:, :, 0:4] = d.view(torch.uint8).view(n, nb, 4)
        return w.view(n, nb * 144)

    def q80(n, k):
        nb = k // 32
        stride = (k + k // 16 + 15) & ~15
        w = torch.zeros((n, stride), dtype=torch.uint8, device=dev)
        w[:, :k] = torch.randint(1, 256, (n, k), dtype=torch.uint8, device=dev, generator=gen)  # int8 in [-127, 127]
        d = (torch.rand((n, nb), device=dev, generator=gen) * (2e-3 - 1e-4) + 1e-4).to(torch.float16)
        w[:, k:k + 2 * nb] = d.view(torch.uint8).view(n, 2 * nb)
        return w

    def quant(ttype, n, k):
        t = q4k(n, k) if ttype == "q4_k" else q80(n, k)
        keep.append(t)
        return (t.data_ptr(), t.numel())

    def vec(n):
        t = (1 + 0.1 * torch.randn(n, device=dev, generator=gen)).float()
        keep.append(t)
        return (t.data_ptr(), t.numel() * 4)

    shapes = layer_weight_shapes(cfg, sh)
    layers = []
    for _ in range(cfg.layers):
        d = {name: quant(cfg.body_type, rows, k) for name, (rows, k) in shapes.items()}
        d["attn_norm"] = vec(cfg.hidden)
        d["ffn_norm"] = vec(cfg.hidden)
        layers.append(d)
    w = {"layers": layers, "embed": quant(cfg.embed_type, cfg.vocab, cfg.hidden),
         "head": quant(cfg.head_type, cfg.vocab // sh.world, cfg.hidden), "out_norm": vec(cfg.hidden)}
    return w, keep


def device_full_model(cfg: DenseConfig, torch, dev, seed: int = 0):
    """A full (unsharded) random model on the device as 2-D uint8 / f32 tensors in the kernels' layouts, the same
    on every rank that calls it with the same seed: what `device_shard` cuts a rank's part out of, so that a
    sharded step and the unsharded step run the SAME model (the parity leg of the multi-GPU bench)."""
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)

    def q4k(n, k):
        nb = k // 256
        w = torch.randint(0, 256, (n, nb, 144), dtype=torch.uint8, device=dev, generator=gen)
        d = (torch.rand((n, nb, 2), device=dev, generator=gen) * (1e-2 - 1e-4) + 1e-4).to(torch.float16)
        w[:, :, 0:4] = d.view(torch.uint8).view(n, nb, 4)
        return w.view(n, nb * 144)

    def q80(n, k):
        nb = k // 32
        stride = (k + k // 16 + 15) & ~15
        w = torch.zeros((n, stride), dtype=torch.uint8, device=dev)
        w[:, :k] = torch.randint(1, 256, (n, k), dtype=torch.uint8, device=dev, generator=gen)
        d = (torch.rand((n, nb), device=dev, generator=gen) * (2e-3 - 1e-4) + 1e-4).to(torch.float16)
        w[:, k:k + 2 * nb] = d.view(torch.uint8).view(n, 2 * nb)
        return w

    def quant(ttype, n, k):
        return q4k(n, k) if ttype == "q4_k" else q80(n, k)

    def vec(n):
        return (1 + 0.1 * torch.randn(n, device=dev, generator=gen)).float()

    layers = []
    for _ in range(cfg.layers):
        layers.append({"wqkv": quant(cfg.body_type, cfg.q_dim + 2 * cfg.kv_dim, cfg.hidden), "wo": quant(cfg.body_type, cfg.hidden, cfg.q_dim),
                       "wgu": quant(cfg.body_type, 2 * cfg.ff, cfg.hidden), "wdown": quant(cfg.body_type, cfg.hidden, cfg.ff),
                       "attn_norm": vec(cfg.hidden), "ffn_norm": vec(cfg.hidden)})
    return {"layers": layers, "embed": quant(cfg.embed_type, cfg.vocab, cfg.hidden), "head": quant(cfg.head_type, cfg.vocab, cfg.hidden),
            "out_norm": vec(cfg.hidden)}


def device_shard(full, cfg: DenseConfig, torch, shard: Shard | None = None):
    """One rank's part of a `device_full_model`, in plan layout: ({name: (ptr, nbytes)}, the tensors that own the
    memory). The rows are the ones `slice_full_weights` names."""
    sh = shard or Shard()
    keep = []
    hd = cfg.head_dim
    h0, h1 = sh.heads(cfg)
    g0, g1 = sh.kv_heads(cfg)
    f0, f1 = shard_rows(cfg.ff, sh.rank, sh.world)
    e0, e1 = shard_rows(cfg.hidden, sh.rank, sh.world)
    v0, v1 = shard_rows(cfg.vocab, sh.rank, sh.world)

    def own(t):
        t = t.contiguous()
        keep.append(t)
        return (t.data_ptr(), t.numel() * t.element_size())

    layers = []
    for lw in full["layers"]:
        w = lw["wqkv"]
        qkv = torch.cat([w[h0 * hd:h1 * hd], w[cfg.q_dim + g0 * hd:cfg.q_dim + g1 * hd],
                         w[cfg.q_dim + cfg.kv_dim + g0 * hd:cfg.q_dim + cfg.kv_dim + g1 * hd]])
        gu = torch.cat([lw["wgu"][f0:f1], lw["wgu"][cfg.ff + f0:cfg.ff + f1]])
        layers.append({"wqkv": own(qkv), "wo": own(lw["wo"][e0:e1]), "wgu": own(gu), "wdown": own(lw["wdown"][e0:e1]),
                       "attn_norm": own(lw["attn_norm"]), "ffn_norm": own(lw["ffn_norm"])})
    return {"layers": layers, "embed": own(full["embed"]), "head": own(full["head"][v0:v1]), "out_norm": own(full["out_norm"])}, keep


def hybrid_host_model(cfg, seed: str = "hybrid"):
    """The full (unsharded) hybrid model on the host: attention layers as host_model's, DeltaNet layers with the
    stacked input projection wproj (rows q | k | v | z | beta | alpha, src/plan/qwen35.zig:556-566), the conv taps
    [channel][tap], dt_bias, a (negative), the gated norm's weight and the output projection."""
    d, hk, hv, taps, e = cfg.gdn_head_dim, cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.conv_kernel, cfg.hidden
    conv_dim = 2 * hk * d + hv * d
    base = host_model(cfg, seed)
    for il in range(cfg.layers):
        if cfg.is_attention(il):
            continue
        r = lambda name: synth.rng_for(seed, f"l{il}.{name}")  # noqa: E731
        lw = base["layers"][il]
        for k in ("wqkv", "wo"):
            del lw[k]
        lw["wproj"] = _quant(r("wproj"), cfg.body_type, conv_dim + hv * d + 2 * hv, e)
        lw["conv"] = (r("conv").uniform(-0.5, 0.5, size=(conv_dim, taps))).astype(np.float32)
        lw["dt_bias"] = r("dt_bias").uniform(-0.5, 0.5, size=hv).astype(np.float32)
        lw["a"] = (-np.abs(r("a").uniform(0.05, 1.0, size=hv))).astype(np.float32)
        lw["norm"] = (1 + 0.1 * r("norm").normal(size=d)).astype(np.float32)
        lw["wout"] = _quant(r("wout"), cfg.body_type, e, hv * d)
    return base


def upload_hybrid(host, cfg, put, shard: Shard | None = None):
    """Device weights of one rank from a hybrid host model."""
    from .plan import slice_delta_weights

    sh = shard or Shard()
    layers = []
    for il, lw in enumerate(host["layers"]):
        d = {"attn_norm": put(lw["attn_norm"]), "ffn_norm": put(lw["ffn_norm"]),
             "wgu": put(slice_full_weights(cfg, sh, "wgu", lw["wgu"])), "wdown": put(slice_full_weights(cfg, sh, "wdown", lw["wdown"]))}
        if cfg.is_attention(il):
            d["wqkv"] = put(slice_full_weights(cfg, sh, "wqkv", lw["wqkv"]))
            d["wo"] = put(slice_full_weights(cfg, sh, "wo", lw["wo"]))
        else:
            for name in ("wproj", "conv", "dt_bias", "a", "wout"):
                d[name] = put(np.ascontiguousarray(slice_delta_weights(cfg, sh, name, lw[name])))
            d["norm"] = put(lw["norm"])
        layers.append(d)
    head = host["head"] if cfg.head_type != "q8_0" else split_q8_0_rows(slice_full_weights(cfg, sh, "head", host["head"]), cfg.hidden)
    return {"layers": layers, "embed": put(host["embed"]), "head": put(head), "out_norm": put(host["out_norm"])}

