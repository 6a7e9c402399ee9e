"""The loader path of the block types beside Q4_K and Q8_0 (Q3_K, Q5_K, Q6_K, IQ4_XS): file blocks laid out for the
kernels (repad / repack_q3_k, src/kernels/repad.wgsl, repack_q3_k.wgsl), table rows decoded bit for bit as the CPU
oracle decodes them (also against the gguf package's vectors), and the decode multiplies against the oracle's
matmul (1e-5 of the f64 sums, 1e-3 of the f32 ones: the bars of src/kernels/check.zig's multiply checks)."""
import numpy as np
import pytest

from tests.util import bits, rel_err
from zllm_b200 import kernels as K
from zllm_b200 import synth

pytestmark = pytest.mark.gpu
TYPES = {"q3_k": "Q3_K", "q5_k": "Q5_K", "q6_k": "Q6_K", "iq4_xs": "IQ4_XS"}


def laid_out(gpu, launcher, ttype, file_rows):
    """The rows in the layout the multiplies read, made on the device from the file bytes."""
    n, nbytes = file_rows.shape
    blocks = n * nbytes // K.FILE_BLOCK[ttype]
    if K.BLOCK_STRIDE[ttype] == K.FILE_BLOCK[ttype]:
        return gpu.put(file_rows)
    dst = gpu.zeros(blocks * K.BLOCK_STRIDE[ttype])
    launcher.layout(ttype, gpu.put(file_rows), dst, blocks)
    return dst


def numpy_repad(file_rows, src, dst):
    blocks = file_rows.reshape(-1, src)
    out = np.zeros((blocks.shape[0], dst), dtype=np.uint8)
    out[:, :src] = blocks
    return out.ravel()


@pytest.mark.parametrize("ttype", ["q6_k", "iq4_xs", "q3_k"])
def test_layout_kernels(gpu, launcher, ttype):
    rng = np.random.default_rng(11)
    rows = synth.kquant_weights(rng, ttype, 3, 256 * 5)   # 15 blocks: odd byte offsets for the 110- and 210-byte blocks
    got = laid_out(gpu, launcher, ttype, rows).download(np.uint8)
    if ttype != "q3_k":
        assert np.array_equal(got, numpy_repad(rows, K.FILE_BLOCK[ttype], K.BLOCK_STRIDE[ttype]))
        return
    # repack_q3_k: unit s of a block = the 2-bit values of half s/4 at bit pair s%4, position 4e + b in byte b of
    # word e/4, bit pair e%4; the high bits one word; the two scales minus 32; d
    blocks = rows.reshape(-1, 110)
    units = got.view(np.uint32).reshape(-1, 8, 4)
    for bi in (0, 7, 14):
        b = blocks[bi]
        for s in range(8):
            half, j = s // 4, s % 4
            l0 = l1 = hw = 0
            for l in range(32):
                q = (int(b[32 + 32 * half + l]) >> (2 * j)) & 3
                h = (int(b[l]) >> (4 * half + j)) & 1
                e, byte = l // 4, l % 4
                if e < 4:
                    l0 |= q << (8 * byte + 2 * e)
                else:
                    l1 |= q << (8 * byte + 2 * (e - 4))
                hw |= h << (8 * byte + e)
            assert [int(x) for x in units[bi, s, :3]] == [l0, l1, hw]
            assert int(units[bi, s, 3]) >> 16 == int(b[108]) | (int(b[109]) << 8)


@pytest.mark.parametrize("ttype", list(TYPES))
def test_embed_rows_are_the_oracle_bits(ref, gpu, launcher, ttype):
    t = getattr(ref, TYPES[ttype])
    g = np.load("tests/golden/dequant_gguf.npz")
    rng = np.random.default_rng(5)
    dim, rows = 512, 40
    table = synth.kquant_weights(rng, ttype, rows, dim, 1e-4, 5e-2, signed_scales=True)
    fb = K.FILE_BLOCK[ttype]
    table[:16] = g[f"{ttype}_bytes"][:32].reshape(16, 2 * fb)      # the gguf package's blocks, edge blocks included
    want = ref.dequantize(t, table, rows * dim).reshape(rows, dim)
    assert np.array_equal(bits(want[:16].ravel()), g[f"{ttype}_f32_bits"][:32].ravel())
    tokens = np.array([0, 1, 39, 7, 15, 200, 3], dtype=np.uint32)   # 200: outside the chunk, its row stays as it was
    # rows as in the file, a stride apart (4 bytes of slack per row)
    stride = table.shape[1] + 4
    padded = np.zeros((rows, stride), dtype=np.uint8)
    padded[:, :table.shape[1]] = table
    for w, st in ((gpu.put(padded), stride), (laid_out(gpu, launcher, ttype, table), 0)):
        out = gpu.put(np.full((tokens.size, dim), 7.0, dtype=np.float32))
        launcher.embed(ttype, gpu.put(tokens), w, out, tokens.size, dim, 0, rows, stride=st)
        got = out.download(np.float32).reshape(tokens.size, dim)
        for i, tok in enumerate(tokens):
            if tok < rows:
                assert np.array_equal(bits(got[i]), bits(want[tok])), (ttype, st, tok)
            else:
                assert (got[i] == 7.0).all()


@pytest.mark.parametrize("ttype", ["q3_k", "q5_k", "q6_k"])
@pytest.mark.parametrize("m", [1, 3])
def test_matvec_matches_the_oracle(ref, gpu, launcher, ttype, m):
    t = getattr(ref, TYPES[ttype])
    rng = synth.rng_for("kquant", f"{ttype}-{m}")
    n, k = 333, 2048                       # a ragged row count; two staged tiles of activations
    file_rows = synth.kquant_weights(rng, ttype, n, k)
    x = rng.normal(size=(m, k)).astype(np.float32)
    w = laid_out(gpu, launcher, ttype, file_rows)
    out = gpu.zeros(m * n * 4)
    launcher.matvec(ttype, gpu.put(x), w, out, n, k, m=m)
    got = out.download(np.float32).reshape(m, n)
    mat = ref.Matrix(t, file_rows, n, k)
    assert rel_err(got, ref.matmul(x, mat, mode=ref.F64)) < 1e-5
    assert rel_err(got, ref.matmul(x, mat)) < 1e-3
    # the fused forms: norm prologue, accumulate
    nw = (1 + 0.1 * rng.normal(size=k)).astype(np.float32)
    base = rng.normal(size=(m, n)).astype(np.float32)
    out2 = gpu.put(base)
    launcher.matvec(ttype, gpu.put(x), w, out2, n, k, m=m, flags=K.NORM | K.ACCUMULATE, eps=1e-6, norm_w=gpu.put(nw))
    h = np.stack([ref.rms_norm(row, nw, 1e-6) for row in x])
    want = base + ref.matmul(h, mat, mode=ref.F64)
    assert rel_err(out2.download(np.float32).reshape(m, n), want) < 1e-5
    # a token's result does not depend on how many tokens the step has
    if m > 1:
        one = gpu.zeros(n * 4)
        launcher.matvec(ttype, gpu.put(x[1]), w, one, n, k, m=1)
        assert np.array_equal(bits(one.download(np.float32)), bits(got[1]))
