"""CPU tier: the C-ABI library loads, exports every declared symbol, and the command-stream interpreter
keeps the reference host's semantics (src/gpu/cmd.zig:285-392, src/agility/host.zig:293-607) in a dry
run, which executes no kernel."""
import re
from pathlib import Path

import numpy as np
import pytest

from zllm_b200 import abi, cmd
from zllm_b200 import kernels as K

ROOT = Path(__file__).resolve().parents[1]


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "zllm_cuda.h").read_text()
    declared = set(re.findall(r"\b(zcu_[a-z_0-9]+)\s*\(", header))
    assert declared == set(abi.EXPORTS)
    L = abi.lib()
    for name in declared:
        assert hasattr(L, name), name


def test_no_device_means_an_error_not_a_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(abi.ZcuError) as e:
        abi.Context(0)
    assert e.value.name == "GpuError"


def test_artifacts_and_missing_kernels():
    for k in (K.MATVEC_Q4_K, K.MATVEC_Q8_0, K.MATVEC_BF16, K.ATTN_SPLIT, K.ATTN_COMBINE, K.DELTA_RULE, K.ROPE_APPEND,
              K.RMSNORM, K.EMBED_Q4_K, K.REPACK_Q8_0, K.MATMUL_BF16, K.QUANTIZE_Q8, K.MATMUL_Q4_K, K.MATMUL_Q8_0,
              K.MATMUL_Q8_0_FLOAT, K.MATMUL_REDUCE, K.SAMPLE, K.MARK_TOKENS, K.DRAFT, K.REPAD, K.REPACK_Q3_K, K.MATVEC_Q3_K,
              K.MATVEC_Q5_K, K.MATVEC_Q6_K, K.EMBED_Q3_K, K.EMBED_Q5_K, K.EMBED_Q6_K, K.EMBED_IQ4_XS):
        assert abi.artifact(k).startswith(b"cuda:")
    for k in (14, 24, 47, 50):  # qsa_keys, gyro_matvec, matmul_q3_k, matmul_q6_k: not on this path
        assert abi.artifact(k) == b""
    for v in K.MATVEC_CANDIDATES:
        assert abi.artifact(K.MATVEC_Q4_K, v)
    assert abi.artifact(K.MATVEC_Q4_K, 0x00012008) == b""  # a WGSL variant id means nothing here
    assert abi.artifact(K.RMSNORM, 5) == b""
    # the reserved prefill-rung id exists for the half-precision multiplies only, and mutated ids do not
    # (src/agility/kernels.zig:200-232)
    for k in (K.MATMUL_BF16, K.MATMUL_F16, K.MATMUL_Q4_K):
        assert abi.artifact(k, K.VARIANT_PREFILL_TC)
        for bit in range(32):
            assert abi.artifact(k, K.VARIANT_PREFILL_TC ^ (1 << bit)) == b""
    assert abi.artifact(K.RMSNORM, K.VARIANT_PREFILL_TC) == b"" and abi.artifact(K.MATMUL_BF16, 0xFFFF0000) == b""
    assert abi.artifact(K.MATMUL_Q8_0, K.VARIANT_PREFILL_TC) == b""
    # the batched tcgen05 family of the decode multiply: Q4_K only, no tile or split bytes
    assert abi.artifact(K.MATVEC_Q4_K, K.MATVEC_BATCHED) == b"cuda:matvec_q4_k:30000"
    assert abi.artifact(K.MATVEC_Q8_0, K.MATVEC_BATCHED) == b"" and abi.artifact(K.MATVEC_Q4_K, K.MATVEC_BATCHED | 4) == b""
    assert K.matvec_variant_exists("q4_k", 4096, K.MATVEC_BATCHED) and not K.matvec_variant_exists("q8_0", 4096, K.MATVEC_BATCHED)
    assert "sm_100a" in abi.backend_source()


@pytest.fixture()
def dry():
    c = abi.Context(dry_run=True)
    yield c
    c.close()


def test_caps_and_budget(dry):
    caps = dry.caps()
    assert caps.abi_version == abi.ABI_VERSION and caps.dry_run == 1 and caps.offset_align == 256
    assert dry.memory_budget() > 0
    assert dry.supports_prefill(0) and dry.supports_prefill(K.VARIANT_PREFILL_TC) and not dry.supports_prefill(0xFFFF0000)


def test_writes_land_before_recorded_work_and_reads_complete(dry):
    r = cmd.Recorder()
    a, b = r.create_buffer(64), r.create_buffer(64)
    r.copy_buffer(a, 0, b, 16, 32)                # recorded first ...
    data = np.arange(16, dtype=np.uint32)
    r.write_buffer(a, 0, data)                    # ... but the write lands before it
    got = np.zeros(16, dtype=np.uint32)
    r.read_buffer(11, b, 0, got)
    r.submit(12)
    assert dry.execute(r.batch()) == [(11, 0), (12, 0)]
    assert got[:4].tolist() == [0] * 4 and got[4:12].tolist() == list(range(8)) and got[12:].tolist() == [0] * 4
    # clear_buffer is ordered with the copies; a submit with no reads reports only itself
    r.clear()
    r.clear_buffer(b, 16, 8)
    r.submit(13)
    got2 = np.zeros(16, dtype=np.uint32)
    r.read_buffer(14, b, 0, got2)
    r.submit(15)
    assert dry.execute(r.batch()) == [(13, 0), (14, 0), (15, 0)]
    assert got2[4:6].tolist() == [0, 0] and got2[6:12].tolist() == list(range(2, 8))


def test_write_file_copies_from_the_mapped_model(dry):
    blob = np.arange(256, dtype=np.uint8)
    dry.set_file(blob, "model.gguf")
    r = cmd.Recorder()
    a = r.create_buffer(64)
    r.write_file(a, 8, 100, 16)
    got = np.zeros(64, dtype=np.uint8)
    r.read_buffer(1, a, 0, got)
    r.submit(2)
    dry.execute(r.batch())
    assert got[8:24].tolist() == list(range(100, 116)) and not got[:8].any() and not got[24:].any()
    r.clear()
    r.write_file(a, 0, 250, 16)  # past the end of the file
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(r.batch())
    assert e.value.name == "BadCommand"


def test_malformed_batches_are_rejected(dry):
    # cmd.Iterator's errors (src/gpu/cmd.zig:222-251)
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(np.array([cmd.SUBMIT | (0 << 8)], dtype=np.uint32))
    assert e.value.name == "BadLength"
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(np.array([cmd.CREATE_BUFFER | (5 << 8), 0, 64], dtype=np.uint32))
    assert e.value.name == "Truncated"
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(np.array([200 | (1 << 8)], dtype=np.uint32))
    assert e.value.name == "BadCommand"
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(np.array([cmd.CREATE_BUFFER | (3 << 8), 0, 64], dtype=np.uint32))  # too few arguments
    assert e.value.name == "BadCommand"
    r = cmd.Recorder()
    r.clear_buffer(5, 0, 4)  # no such buffer
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(r.batch())
    assert e.value.name == "BadId"
    r.clear()
    a = r.create_buffer(16)
    r.copy_buffer(a, 0, a, 8, 16)  # runs past the buffer
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(r.batch())
    assert e.value.name == "BadCommand"
    r.clear()
    r.write_buffer(a, 2, np.zeros(1, dtype=np.uint32))  # offset not a multiple of 4
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(r.batch())
    assert e.value.name == "BadCommand"


def test_missing_kernel_fails_the_batch_and_drops_the_submission(dry):
    r = cmd.Recorder()
    a = r.create_buffer(64)
    missing = r.create_kernel(22, 0, 0, b"")      # `sample`: empty artifact = not implemented
    real = r.create_kernel(K.SILU_MUL, 0, 1 << 2, abi.artifact(K.SILU_MUL))
    dry.execute(r.batch())
    r.clear()
    r.write_buffer(a, 0, np.full(16, 7, dtype=np.uint32))
    r.dispatch(missing, (1, 1, 1), [])
    r.submit(1)
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(r.batch())
    assert e.value.name == "UnsupportedKernel" and e.value.completions == []
    # the staged write was dropped with the submission
    r.clear()
    got = np.ones(16, dtype=np.uint32)
    r.read_buffer(2, a, 0, got)
    r.submit(3)
    assert dry.execute(r.batch()) == [(2, 0), (3, 0)]
    assert not got.any()
    # a pipeline of this backend dispatches (counted, not executed, in a dry run)
    before = dry.launch_count()
    page = np.frombuffer(bytes(K.SiluMul(8, 8)), dtype=np.uint8)
    r.clear()
    u = r.create_buffer(256, cmd.UNIFORM | cmd.COPY_DST)
    g = r.create_bind_group(real, [(0, u, 0, 16), (1, a, 0, 64), (2, a, 0, 32)])
    r.write_buffer(u, 0, page)
    r.dispatch(real, (1, 1, 1), [g])
    r.submit(4)
    assert dry.execute(r.batch()) == [(4, 0)]
    assert dry.launch_count() == before + 1
    # creating a pipeline of an identity the backend lacks, with a non-empty artifact, is refused
    r.clear()
    r.create_kernel(24, 0, 0, b"cuda:gyro_matvec")
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(r.batch())
    assert e.value.name == "UnsupportedKernel"


def test_destroy_and_id_reuse(dry):
    r = cmd.Recorder()
    a = r.create_buffer(32)
    r.destroy(cmd.KIND_BUFFER, a)
    r.clear_buffer(a, 0, 4)
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(r.batch())
    assert e.value.name == "BadId"
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(np.array([cmd.CREATE_BUFFER | (5 << 8), 1, 64, 0, 0, cmd.CREATE_BUFFER | (5 << 8), 1, 64, 0, 0],
                             dtype=np.uint32))
    assert e.value.name == "BadId"  # id 1 created twice


def test_forced_loss_is_a_host_flag(dry):
    dry.force_loss()
    with pytest.raises(abi.ZcuError) as e:
        dry.execute(np.array([cmd.SUBMIT | (2 << 8), 1], dtype=np.uint32))
    assert e.value.name == "DeviceLost"
    with pytest.raises(abi.ZcuError):
        dry.alloc(16)


def test_recorder_round_trip():
    # src/gpu/cmd.zig:285-330: every command decodes to what was recorded.
    r = cmd.Recorder()
    b0 = r.create_buffer((5 << 32) | 7, cmd.STORAGE)
    data = np.arange(4, dtype=np.uint32)
    r.write_buffer(b0, 8, data)
    p = r.create_kernel(K.RMSNORM, 0, 8, b"cuda:rmsnorm")
    g = r.create_bind_group(p, [(0, b0, 0, 16), (3, b0, 256, 1 << 33)])
    r.dispatch(p, (3, 2, 1), [g])
    r.submit(42)
    ops = list(cmd.iterate(r.batch()))
    assert [o for o, _ in ops] == [cmd.CREATE_BUFFER, cmd.WRITE_BUFFER, cmd.CREATE_KERNEL, cmd.CREATE_BIND_GROUP,
                                   cmd.DISPATCH, cmd.SUBMIT]
    assert ops[0][1] == [0, 7, 5, cmd.STORAGE]
    assert ops[1][1][:3] == [0, 8, 0] and ops[1][1][5:] == [16, 0]
    assert ops[3][1][:4] == [0, 0, 0, 2] and ops[3][1][10:] == [3, 0, 256, 0, 0, 2]
    assert ops[4][1] == [0, 3, 2, 1, 1, 0] and ops[5][1] == [42]
    assert (r.next == [1, 1, 1])
    with pytest.raises(ValueError):
        list(cmd.iterate(r.batch()[:-1]))


def test_the_default_form_named_in_the_header_is_the_one_the_tuning_skips():
    # Variant word 0 of matvec_q4_k resolves to one of the sweep's candidates; the in-step trials must know which, so
    # that they do not time the default against itself. The header states it; the host mirror and the library agree.
    root = Path(__file__).resolve().parent.parent
    text = (root / "include" / "zllm_cuda.h").read_text()
    m = re.search(r"matvec_q4_k is ZCU_VARIANT\((\d+), (0x[0-9a-f]+), ZCU_FAMILY_MMA\)", text)
    assert m, "the header no longer states matvec_q4_k's default form"
    stated = K.variant(int(m.group(1)), int(m.group(2), 16), K.FAMILY_MMA)
    assert stated == K.MATVEC_DEFAULT_FORM["q4_k"] and stated in K.MATVEC_CANDIDATES
    src = (root / "zllm_b200" / "csrc" / "k_matvec.cu").read_text()
    assert f"launch_matvec_imma(a, v, TYPE, {m.group(1)}, {m.group(2)})" in src
