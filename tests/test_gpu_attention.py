"""Parity of rope_append, attn_split and attn_combine with the CPU oracle (src/ref/dense.zig:201-280,
src/ref/qwen35.zig:331-420), through the C ABI. Case designs follow src/kernels/check.zig:1478-1559."""
import math

import numpy as np
import pytest

from tests.util import bits, rel_err, uniform
from zllm_b200 import kernels as K
from zllm_b200 import synth

pytestmark = pytest.mark.gpu
TOL = 1e-5


def run_attention(gpu, launcher, q_rows, kc, vc, pos0, heads, kv_heads, hd, gated, kv_fmt, max_keys, variant=0):
    """q_rows: [m, q_row] f32 (heads interleaved with gates when gated). Returns out [m, heads, hd]."""
    m, q_row = q_rows.shape
    max_blocks = -(-max_keys // K.ATTN_BLOCK)
    p = K.Attention(heads, kv_heads, hd, kv_fmt, K.attention_scale(hd), max_blocks, q_row, 0, int(gated), 0)
    part = gpu.zeros(m * heads * max_blocks * (hd + 2) * 4)
    out = gpu.zeros(m * heads * hd * 4)
    step = gpu.put(np.array([m, pos0, 0, 0], dtype=np.uint32))
    dq, dk, dv = gpu.put(q_rows), gpu.put(kc), gpu.put(vc)
    launcher.attn_split(p, dq, dk, dv, part, step, pos0 + m, m, variant=variant)
    launcher.attn_combine(p, dq, part, out, step, m)
    return out.download(np.float32).reshape(m, heads, hd)


@pytest.mark.parametrize("heads,kv_heads,hd,gated", [(8, 2, 256, True), (12, 1, 256, False), (32, 8, 128, False),
                                                     (4, 4, 64, True)])
def test_attn_decode_f16_cache(ref, gpu, launcher, heads, kv_heads, hd, gated):
    # 3 queries after 150 positions: 3 blocks, the last partial; groups 4 and 12; gated and ungated.
    rng = np.random.default_rng(heads * 1000 + hd)
    pos0, m = 150, 3
    keys_max = pos0 + m
    kcf = uniform(rng, (keys_max, kv_heads, hd), 1.0).astype(np.float16)
    vcf = uniform(rng, (keys_max, kv_heads, hd), 1.0).astype(np.float16)
    q_head = 2 * hd if gated else hd
    q_rows = uniform(rng, (m, heads * q_head), 1.0)
    fast = heads // kv_heads <= 4 and hd in (64, 128)
    for variant in ((0, 1, 3) if fast else (0,)):  # both arithmetics of the fast path; the generic path otherwise
        got = run_attention(gpu, launcher, q_rows, kcf.view(np.uint16), vcf.view(np.uint16), pos0, heads, kv_heads, hd,
                            gated, K.KV_F16, 256, variant=variant)
        _check_rows(ref, got, q_rows, kcf, vcf, pos0, m, heads, kv_heads, hd, gated, q_head)


def _check_rows(ref, got, q_rows, kcf, vcf, pos0, m, heads, kv_heads, hd, gated, q_head):
    for t in range(m):
        qv = q_rows[t].reshape(heads, q_head)
        gate = qv[:, hd:] if gated else None
        want = ref.attend_decode(qv[:, :hd].copy(), kcf.view(np.uint16), vcf.view(np.uint16), pos0 + t + 1, heads,
                                 kv_heads, hd, K.attention_scale(hd), gate=None if gate is None else gate.copy())
        assert rel_err(got[t], want) < TOL, (t, rel_err(got[t], want))


def test_attn_decode_f32_cache_and_single_key(ref, gpu, launcher):
    rng = np.random.default_rng(5)
    heads, kv_heads, hd = 4, 2, 64
    kcf = uniform(rng, (70, kv_heads, hd), 1.0)
    vcf = uniform(rng, (70, kv_heads, hd), 1.0)
    q_rows = uniform(rng, (1, heads * hd), 1.0)
    # one key: the output is V itself
    got = run_attention(gpu, launcher, q_rows, kcf, vcf, 0, heads, kv_heads, hd, False, K.KV_F32, 128)
    for h in range(heads):
        assert np.abs(got[0, h] - vcf[0, h // 2]).max() < 1e-6
    # 70 keys, f32 cache, against float64
    got = run_attention(gpu, launcher, q_rows, kcf, vcf, 69, heads, kv_heads, hd, False, K.KV_F32, 128)
    for h in range(heads):
        s = kcf[:, h // 2].astype(np.float64) @ q_rows[0].reshape(heads, hd)[h].astype(np.float64) / math.sqrt(hd)
        pr = np.exp(s - s.max())
        want = (pr[:, None] * vcf[:, h // 2].astype(np.float64)).sum(0) / pr.sum()
        assert rel_err(got[0, h], want) < TOL


def test_attn_decode_llama_shape_8192(ref, gpu, launcher):
    # The decode-step configuration: 32 query / 8 KV heads of 128, f16 cache ~ N(0,1) with 8192 positions.
    rng = synth.rng_for("cfg5", "kv0")
    heads, kv_heads, hd, pos0 = 32, 8, 128, 8192
    kcf = rng.normal(size=(pos0 + 1, kv_heads, hd)).astype(np.float16)
    vcf = rng.normal(size=(pos0 + 1, kv_heads, hd)).astype(np.float16)
    q = rng.normal(size=(1, heads * hd)).astype(np.float32)
    got = run_attention(gpu, launcher, q, kcf.view(np.uint16), vcf.view(np.uint16), pos0, heads, kv_heads, hd, False,
                        K.KV_F16, pos0 + 1)
    want = ref.attend_decode(q.reshape(heads, hd), kcf.view(np.uint16), vcf.view(np.uint16), pos0 + 1, heads, kv_heads,
                             hd, K.attention_scale(hd))
    assert rel_err(got[0], want) < TOL


@pytest.mark.parametrize("normal,qk_norm,gated", [(1, 0, 0), (0, 1, 1)])
def test_rope_append_writes_rounded_cache(ref, gpu, launcher, normal, qk_norm, gated):
    # Llama style (normal pairs, no Q/K norm, ungated) and Qwen style (NeoX, per-head norm, gated).
    rng = np.random.default_rng(21 + normal)
    heads, kv_heads, hd, n_rot, base, eps = 4, 2, 64, 64 if normal else 32, 500000.0 if normal else 10000.0, 1e-6
    m, pos0, max_pos = 3, 5, 16
    q_head = 2 * hd if gated else hd
    k_off = heads * q_head
    v_off = k_off + kv_heads * hd
    row = v_off + kv_heads * hd
    qkv = uniform(rng, (m, row), 2.0)
    qn, kn = uniform(rng, hd, 1.5), uniform(rng, hd, 1.5)
    table = ref.rope_table(max_pos, n_rot, base)
    for kv_fmt in (K.KV_F16, K.KV_F32):
        width = kv_heads * hd
        cache_words = max_pos * width // (2 if kv_fmt == K.KV_F16 else 1)
        kc, vc = gpu.zeros(cache_words * 4), gpu.zeros(cache_words * 4)
        dq = gpu.put(qkv)
        p = K.RopeAppend(heads, kv_heads, hd, n_rot, row, k_off, v_off, kv_fmt, eps, gated, qk_norm, normal, 0)
        step = gpu.put(np.array([m, pos0, 0, 0], dtype=np.uint32))
        launcher.rope_append(p, dq, gpu.put(qn), gpu.put(kn), gpu.put(table), kc, vc, step, m)
        got = dq.download(np.float32).reshape(m, row)
        kcache = kc.download(np.uint16 if kv_fmt == K.KV_F16 else np.float32).reshape(max_pos, kv_heads, hd)
        vcache = vc.download(np.uint16 if kv_fmt == K.KV_F16 else np.float32).reshape(max_pos, kv_heads, hd)
        for t in range(m):
            pos = pos0 + t

            def prep(vec, w):
                if qk_norm:
                    vec = ref.rms_norm(vec, w, eps)
                return ref.rope_normal(vec, pos, n_rot, base) if normal else ref.rope(vec, pos, n_rot, base)

            for h in range(heads):
                want = prep(qkv[t, h * q_head:h * q_head + hd], qn)
                g = got[t, h * q_head:h * q_head + hd]
                if qk_norm:
                    assert rel_err(g, want) < 1e-6
                else:
                    assert np.array_equal(bits(g), bits(want))  # same products, same roundings
                if gated:  # the gate half is untouched
                    assert np.array_equal(got[t, h * q_head + hd:(h + 1) * q_head], qkv[t, h * q_head + hd:(h + 1) * q_head])
            for g_ in range(kv_heads):
                wk = prep(qkv[t, k_off + g_ * hd:k_off + (g_ + 1) * hd], kn)
                wv = qkv[t, v_off + g_ * hd:v_off + (g_ + 1) * hd]
                if kv_fmt == K.KV_F16:
                    assert np.array_equal(vcache[pos, g_], ref.to_f16_bits(wv))  # RNE, bit for bit
                    if not qk_norm:
                        assert np.array_equal(kcache[pos, g_], ref.to_f16_bits(wk))
                    else:
                        assert rel_err(kcache[pos, g_].view(np.float16).astype(np.float32), wk) < 1e-3
                else:
                    assert np.array_equal(bits(vcache[pos, g_]), bits(wv))
                    assert rel_err(kcache[pos, g_], wk) < 1e-6
        # positions outside the step stay zero
        assert not kcache[:pos0].any() and not kcache[pos0 + m:].any()


def test_both_arithmetics_of_the_split_agree(gpu, launcher):
    # The CUDA-core form (variant 1: exact f32 products) and the tensor-core form (variant 3 = the default: queries
    # and probabilities as two f16 terms) agree, for rows with different key counts (batched sequences: 700, 1 and
    # 333 keys, so some blocks hold no keys at all and some warps of a block hold none).
    rng = np.random.default_rng(91)
    heads, kv_heads, hd, rows, ctx = 8, 2, 128, 3, 768
    positions = np.array([699, 0, 332], dtype=np.uint32)
    kc = rng.normal(size=(rows, ctx, kv_heads, hd)).astype(np.float16)
    vc = rng.normal(size=(rows, ctx, kv_heads, hd)).astype(np.float16)
    q = uniform(rng, (rows, heads * hd), 1.0)
    max_blocks = -(-ctx // K.ATTN_BLOCK)
    p = K.Attention(heads, kv_heads, hd, K.KV_F16, K.attention_scale(hd), max_blocks, heads * hd, 0, 0, 0)
    p._pad[0] = ctx * kv_heads * hd
    dq, dk, dv = gpu.put(q), gpu.put(kc.view(np.uint16)), gpu.put(vc.view(np.uint16))
    step, dpos = gpu.put(np.array([rows, 0, 0, 0], dtype=np.uint32)), gpu.put(positions)
    got = []
    for variant in (1, 3):
        part = gpu.zeros(rows * heads * max_blocks * (hd + 2) * 4)
        out = gpu.zeros(rows * heads * hd * 4)
        launcher.launch(K.ATTN_SPLIT, p, [dq, dk, dv, part, step, dpos], (kv_heads, max_blocks, rows), variant)
        launcher.launch(K.ATTN_COMBINE, p, [dq, part, out, step, dpos], (heads, rows, 1))
        gpu.sync()
        got.append((part.download(np.uint32), out.download(np.uint32)))
    assert np.abs(got[0][1].view(np.float32)).max() > 0
    pa = got[0][0].view(np.float32).reshape(rows, heads, max_blocks, hd + 2)
    for other in got[1:]:   # the tensor-core forms (K staged in shared memory, K through registers) against the CUDA-core form
        assert rel_err(other[1].view(np.float32), got[0][1].view(np.float32)) < TOL
        # a block's partial {max, sum exp, sum exp * v} is the same softmax state in every form
        pb = other[0].view(np.float32).reshape(rows, heads, max_blocks, hd + 2)
        for t in range(rows):
            used = -(-(int(positions[t]) + 1) // 128)
            assert rel_err(pb[t, :, :used, 0], pa[t, :, :used, 0]) < TOL and rel_err(pb[t, :, :used, 1:], pa[t, :, :used, 1:]) < TOL, t


def test_fp8_cache_append_and_attention(ref, gpu, launcher):
    # The FP8 KV cache (src/ref/fp8.zig, src/kernels/fp8.wgsl): rope_append stores each (position, KV head) row as
    # E4M3FN bytes over a power-of-two scale kept as f32 after the values; attention reads value * scale. The bytes
    # and scales are the codec oracle's, bit for bit (Llama style: no norm, so K before rounding is bit-equal too);
    # attention over the cache then matches the oracle's attention over the decoded values.
    from oracle import sampler as S

    rng = np.random.default_rng(77)
    heads, kv_heads, hd, n_rot, base = 8, 2, 128, 128, 500000.0
    m, pos0, max_pos = 3, 70, 128
    k_off = heads * hd
    v_off = k_off + kv_heads * hd
    row = v_off + kv_heads * hd
    width = kv_heads * hd
    scales = max_pos * width // 4                        # the scales follow the values, in words
    words = scales + max_pos * kv_heads
    table = ref.rope_table(max_pos, n_rot, base)
    # a cache of earlier positions: rows of widely different magnitudes, encoded by the oracle
    kq, vq = np.zeros(words, dtype=np.uint32), np.zeros(words, dtype=np.uint32)
    kdec = np.zeros((max_pos, kv_heads, hd), dtype=np.float32)
    vdec = np.zeros((max_pos, kv_heads, hd), dtype=np.float32)

    def store(cache, dec, pos, g, vec):
        s = S.fp8_row_scale(vec)
        codes = np.array([S.fp8_encode(x / s) for x in vec], dtype=np.uint8)
        cache.view(np.uint8)[(pos * width + g * hd):(pos * width + (g + 1) * hd)] = codes
        cache[scales + pos * kv_heads + g] = np.float32(s).view(np.uint32)
        dec[pos, g] = S.FP8_TABLE[codes] * np.float32(s)

    for pos in range(pos0):
        for g in range(kv_heads):
            store(kq, kdec, pos, g, (rng.normal(size=hd) * 10.0 ** rng.uniform(-2, 2)).astype(np.float32))
            store(vq, vdec, pos, g, (rng.normal(size=hd) * 10.0 ** rng.uniform(-2, 2)).astype(np.float32))
    qkv = uniform(rng, (m, row), 3.0)
    qkv[1, k_off:k_off + hd] = 0.0                       # a zero K row: scale 1
    dq, kc, vc = gpu.put(qkv), gpu.put(kq), gpu.put(vq)
    p = K.RopeAppend(heads, kv_heads, hd, n_rot, row, k_off, v_off, K.KV_FP8, 1e-6, 0, 0, 1, scales)
    step = gpu.put(np.array([m, pos0, 0, 0], dtype=np.uint32))
    one = gpu.put(np.ones(hd, dtype=np.float32))
    launcher.rope_append(p, dq, one, one, gpu.put(table), kc, vc, step, m)
    gpu.sync()
    got_k, got_v = kc.download(np.uint32), vc.download(np.uint32)
    for t in range(m):
        for g in range(kv_heads):
            store(kq, kdec, pos0 + t, g, ref.rope_normal(qkv[t, k_off + g * hd:k_off + (g + 1) * hd], pos0 + t, n_rot, base))
            store(vq, vdec, pos0 + t, g, qkv[t, v_off + g * hd:v_off + (g + 1) * hd])
    assert np.array_equal(got_k, kq) and np.array_equal(got_v, vq)
    assert kq[scales + (pos0 + 1) * kv_heads] == np.float32(1).view(np.uint32)
    # attention over the FP8 cache (the queries rope_append rotated in place)
    q_rows = dq.download(np.float32).reshape(m, row)[:, :heads * hd].copy()
    max_blocks = -(-max_pos // K.ATTN_BLOCK)
    ap = K.Attention(heads, kv_heads, hd, K.KV_FP8, K.attention_scale(hd), max_blocks, heads * hd, 0, 0, scales)
    part, out = gpu.zeros(m * heads * max_blocks * (hd + 2) * 4), gpu.zeros(m * heads * hd * 4)
    dqr = gpu.put(q_rows)
    launcher.attn_split(ap, dqr, kc, vc, part, step, pos0 + m, m)
    launcher.attn_combine(ap, dqr, part, out, step, m)
    got = out.download(np.float32).reshape(m, heads, hd)
    for t in range(m):
        n = pos0 + t + 1
        for h in range(heads):
            g = h // (heads // kv_heads)
            s = kdec[:n, g].astype(np.float64) @ q_rows[t].reshape(heads, hd)[h].astype(np.float64) / math.sqrt(hd)
            pr = np.exp(s - s.max())
            want = (pr[:, None] * vdec[:n, g].astype(np.float64)).sum(0) / pr.sum()
            assert rel_err(got[t, h], want) < TOL, (t, h, rel_err(got[t, h], want))
