"""Writes the golden fixtures of this directory.

reference_kats.json
    Known-answer values transcribed from the reference's own unit tests (values
    only): the E4M3 codec cases of src/backend/vulkan/fp8_ext.rs:225-263, the
    layout integers of src/backend/vulkan/kv_cache.rs:519-586, and the edge list
    the codec must honour.  The Rust reference cannot be compiled here (no cargo),
    so these are the machine-checkable anchors it offers for this path.
attention_small.npz
    The CPU oracle's outputs for a few small seeded attention cases, so the GPU
    tests can also be checked against committed numbers.  Inputs are regenerated
    from the seed by util.golden_inputs; a CRC of the input bytes is stored to
    detect generator drift.

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from util import GOLDEN_CASES, golden_inputs  # noqa: E402

KATS = {
    "e4m3_encode": [  # [f32 value, code]  fp8_ext.rs:225-249
        [0.0, 0x00], [-0.0, 0x80], [1.0, 0x38], [448.0, 0x7E], [1000.0, 0x7E],
    ],
    "e4m3_decode": [  # [code, f32 value]  fp8_ext.rs:228-262
        [0x00, 0.0], [0x80, -0.0], [0x38, 1.0], [0x7E, 448.0], [0x40, 2.0], [0x48, 4.0],
        [0xB8, -1.0], [0x30, 0.5], [0x3C, 1.5],
    ],
    # consequences of fp8_ext.rs:126-187 at the edges (saturation, ties, subnormals)
    "e4m3_edges": [
        [464.0, 0x7E], [-464.0, 0xFE], [447.9, 0x7E], [432.0, 0x7E], [440.0, 0x7E], [424.0, 0x7D], [400.0, 0x7C],
        [0.001953125, 0x01], [0.0009765625, 0x00], [0.00146484375, 0x01], [0.0029296875, 0x02],
        [0.015625, 0x08], [0.0146484375, 0x08], [1e-45, 0x00], [-1e-45, 0x80],
        ["inf", 0x7E], ["-inf", 0xFE], ["nan", 0x7F], ["-nan", 0x7F],
    ],
    "layout": {  # kv_cache.rs:519-586
        "bytes_per_token_uniform_f16": {"n_layers": 40, "n_kv_heads": 8, "head_dim": 128, "elem": 2,
                                        "expect": 2 * 2 * 40 * 8 * 128},
        "bytes_per_token_hetero_fp8": {"plhd": [256, 256, 512, 512], "plkv": [2, 2, 4, 4], "elem": 1,
                                       "expect": 10240},
        "qwen3_8b_f32_total": {"n_layers": 36, "n_kv_heads": 8, "head_dim": 128, "max_seq": 2048,
                               "expect_bytes": 576 * 1024 * 1024},
        "qwen3_8b_f16_total": {"n_layers": 36, "n_kv_heads": 8, "head_dim": 128, "max_seq": 2048,
                               "expect_bytes": 288 * 1024 * 1024},
    },
}


def attention_cases():
    import zlib
    out = {}
    for i, (name, hq, hkv, d, L, start, dt, cap) in enumerate(GOLDEN_CASES):
        q, kc, vc = golden_inputs(i)
        o = oracle.attention_ref(q, kc, vc, dt, hq, hkv, d, L, start, None, cap)
        crc = zlib.crc32(q.tobytes()) ^ zlib.crc32(kc.tobytes()) ^ zlib.crc32(vc.tobytes())
        out[name + "/crc"] = np.uint32(crc)
        out[name + "/out"] = o
    return out


if __name__ == "__main__":
    with open(os.path.join(HERE, "reference_kats.json"), "w") as f:
        json.dump(KATS, f, indent=1)
    np.savez_compressed(os.path.join(HERE, "attention_small.npz"), **attention_cases())
    print("wrote", os.listdir(HERE))
