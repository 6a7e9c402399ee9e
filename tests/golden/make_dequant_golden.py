"""Makes tests/golden/dequant_gguf.npz: random Q8_0, Q4_K, Q3_K, Q5_K, Q6_K and IQ4_XS blocks and their
f32 decodings by the numpy dequantisers of the `gguf` Python package (an
implementation of ggml's dequantize_row_* independent of both the reference
and this repository). The reference states bitwise agreement with ggml for
these block types (src/ref/tensor.zig:17-20) but carries no known-answer vector
for them, so these fixtures are the pin. Run from the repository root:

    python tests/golden/make_dequant_golden.py
"""
import sys
from pathlib import Path

import numpy as np
from gguf import GGMLQuantizationType as T
from gguf import quants

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from zllm_b200 import synth  # noqa: E402


def main() -> None:
    rng = np.random.default_rng(0x5EED)
    q8 = synth.q8_0_weights(rng, 4, 32 * 24, 1e-4, 5e-2, signed_scales=True)
    q4 = synth.q4_k_weights(rng, 4, 256 * 12, 1e-4, 5e-2, signed_scales=True)
    # Edge blocks: all-zero bytes, all-ones bytes, extreme nibbles/scales.
    q4[0, :144] = 0
    q4[0, 144:288] = 0xFF
    q4[0, 144:148] = np.array([0.0078125, -0.001953125], dtype=np.float16).view(np.uint8)
    q8[0, :34] = 0
    q8[0, 34:68] = 0x80
    q8[0, 34:36] = np.array([-0.0009765625], dtype=np.float16).view(np.uint8)
    out8 = quants.dequantize(q8.reshape(-1, 34), T.Q8_0).astype(np.float32)
    out4 = quants.dequantize(q4.reshape(-1, 144), T.Q4_K).astype(np.float32)
    more = {}
    for name, tt in (("q3_k", T.Q3_K), ("q5_k", T.Q5_K), ("q6_k", T.Q6_K), ("iq4_xs", T.IQ4_XS)):
        bb = synth.KQUANT_BLOCK_BYTES[name]
        w = synth.kquant_weights(rng, name, 4, 256 * 8, 1e-4, 5e-2, signed_scales=True)
        w[0, :bb] = 0                      # edge blocks: all-zero and all-ones bytes (with a finite super-scale)
        w[0, bb:2 * bb] = 0xFF
        for at in synth._KQUANT_D_AT[name]:
            w[0, bb + at:bb + at + 2] = np.array([-0.001953125], dtype=np.float16).view(np.uint8)
        out = quants.dequantize(w.reshape(-1, bb), tt).astype(np.float32)
        more[f"{name}_bytes"], more[f"{name}_f32_bits"] = w.reshape(-1, bb), out.view(np.uint32)
        print(name, "blocks", out.shape)
    np.savez_compressed(Path(__file__).with_name("dequant_gguf.npz"), q8_0_bytes=q8.reshape(-1, 34),
                        q8_0_f32_bits=out8.view(np.uint32), q4_k_bytes=q4.reshape(-1, 144),
                        q4_k_f32_bits=out4.view(np.uint32), **more)
    print("q8_0 blocks", out8.shape, "q4_k blocks", out4.shape)


if __name__ == "__main__":
    main()
