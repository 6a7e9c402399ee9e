"""The allocation-free decode-attention entry point (zcu_attention_decode_static) against the ordinary
attn_split + attn_combine pair, through the C ABI. Some hosts of this library cannot call cudaMalloc (they
are given input and output buffers and no budget of their own, or sit on a path where an allocation's
implicit synchronisation is not allowed); for them the per-block partials live in a fixed array inside the
library. Two calls in a row are checked, because every call shares that array and it keeps what the last
call left there. This file sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import numpy as np
import pytest

from zllm_b200 import abi
from zllm_b200 import kernels as K

pytestmark = pytest.mark.gpu


def _case(gpu, launcher, rng, heads, kv_heads, hd, pos0, rows, gated):
    keys_max = pos0 + rows
    kc = rng.normal(size=(keys_max, kv_heads, hd)).astype(np.float16).view(np.uint16)
    vc = rng.normal(size=(keys_max, kv_heads, hd)).astype(np.float16).view(np.uint16)
    q_head = 2 * hd if gated else hd
    q = rng.normal(size=(rows, heads * q_head)).astype(np.float32)
    dq, dk, dv = gpu.put(q), gpu.put(kc), gpu.put(vc)
    step = gpu.put(np.array([rows, pos0, 0, 0], dtype=np.uint32))
    max_blocks = -(-keys_max // K.ATTN_BLOCK)
    p = K.Attention(heads, kv_heads, hd, K.KV_F16, K.attention_scale(hd), max_blocks, heads * q_head, 0, int(gated), 0)
    # the existing entry point: partials in a buffer the caller allocates
    part = gpu.zeros(rows * heads * max_blocks * (hd + 2) * 4)
    want = gpu.zeros(rows * heads * hd * 4)
    launcher.attn_split(p, dq, dk, dv, part, step, keys_max, rows)
    launcher.attn_combine(p, dq, part, want, step, rows)
    # the allocation-free one: same inputs, same output buffer shape, nothing else
    got = gpu.zeros(rows * heads * hd * 4)
    gpu.attention_decode_static(p, [dq, dk, dv, got, step], keys_max, rows)
    a, b = got.download(np.float32), want.download(np.float32)
    assert np.isfinite(b).all() and np.abs(b).max() > 0
    assert np.abs(a - b).max() <= 1e-5 * np.abs(b).max()  # the tolerance of the attention parity tests
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))  # in fact the same kernels: the same bits


def test_static_partials_match_the_allocating_path_on_two_calls_in_a_row(gpu, launcher):
    rng = np.random.default_rng(2024)
    # first call: the Llama-shaped fast path (f16 cache, group 4, head_dim 128), three blocks of keys
    _case(gpu, launcher, rng, heads=32, kv_heads=8, hd=128, pos0=300, rows=1, gated=False)
    # second call, straight after, with a different shape: it finds the first call's partials in the array
    # and must not be affected by them (the generic path: gated, head_dim 256, group 4, 3 rows)
    _case(gpu, launcher, rng, heads=8, kv_heads=2, hd=256, pos0=150, rows=3, gated=True)
    # and the first shape again
    _case(gpu, launcher, rng, heads=32, kv_heads=8, hd=128, pos0=299, rows=2, gated=False)


def test_static_partials_reject_sizes_beyond_the_fixed_array(gpu):
    heads, kv_heads, hd = 64, 8, 128
    p = K.Attention(heads, kv_heads, hd, K.KV_F16, K.attention_scale(hd), 0, heads * hd, 0, 0, 0)
    dummy = gpu.zeros(256)
    with pytest.raises(abi.ZcuError) as e:
        # 64 heads x ceil(20000 / 64) blocks x 130 floats = 2.6 M floats > 1 Mi: refused before anything is launched
        gpu.attention_decode_static(p, [dummy, dummy, dummy, dummy, dummy], 20000, 1)
    assert e.value.name == "Invalid" and "4 MiB" in e.value.message
    gpu.sync()  # the context is still usable


def test_a_step_past_max_keys_is_reported_not_followed(gpu, launcher):
    # max_keys is fixed when the call is made (or captured) while the Step buffer moves on with every replay: a
    # position past what the call covers must neither read past the cache nor past the fixed array - the kernels
    # leave the keys beyond out and the next sync says so.
    rng = np.random.default_rng(77)
    heads, kv_heads, hd, max_keys = 32, 8, 128, 256
    kc = rng.normal(size=(max_keys, kv_heads, hd)).astype(np.float16).view(np.uint16)
    vc = rng.normal(size=(max_keys, kv_heads, hd)).astype(np.float16).view(np.uint16)
    q = rng.normal(size=(1, heads * hd)).astype(np.float32)
    dq, dk, dv, out = gpu.put(q), gpu.put(kc), gpu.put(vc), gpu.zeros(heads * hd * 4)
    p = K.Attention(heads, kv_heads, hd, K.KV_F16, K.attention_scale(hd), 0, heads * hd, 0, 0, 0)
    step = gpu.put(np.array([1, 5000, 0, 0], dtype=np.uint32))   # position 5000, cache and call cover 256 keys
    gpu.attention_decode_static(p, [dq, dk, dv, out, step], max_keys, 1)
    with pytest.raises(abi.ZcuError) as e:
        gpu.sync()
    assert e.value.name == "GpuError" and "past the key blocks" in e.value.message
    # the same call with the Step inside the range works, and the context is intact
    step = gpu.put(np.array([1, max_keys - 1, 0, 0], dtype=np.uint32))
    gpu.attention_decode_static(p, [dq, dk, dv, out, step], max_keys, 1)
    gpu.sync()
    assert np.isfinite(out.download(np.float32)).all() and np.abs(out.download(np.float32)).max() > 0

