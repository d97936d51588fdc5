#!/usr/bin/env python
"""Regenerates the golden vectors under tests/golden/ (run where the reference tree and gguf-py are present).

Sources of truth, none of them this repository's own code:
  * the reference's three I2_S fixtures (tests/fixtures/*.bin of uno-km/ameva-compute) with the SHA-256 values its
    fixture_manifest.json records — copied verbatim (224 bytes in total);
  * gguf-py (the Python package of the llama.cpp project, version recorded in the output): Q8_0 / Q4_0 quantizers that
    describe themselves as bit-exact with ggml's reference quantizers, and the Q4_0 / Q8_0 / Q4_K dequantizers;
  * the reference's own I2_S CPU dot kernel (adapters/bitnet/src/cpu/ggml_bitnet_mad.cpp, scalar branch), compiled by
    oracle/Makefile into oracle/_ref/libbitnet_ref.so and called on seeded inputs.

Usage:  python tests/golden/make_golden.py [--reference <checkout of uno-km/ameva-compute>]
"""
import argparse
import hashlib
import json
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("AMEVA_REFERENCE_ROOT"), required="AMEVA_REFERENCE_ROOT" not in os.environ,
                    help="a checkout of uno-km/ameva-compute (or the AMEVA_REFERENCE_ROOT environment variable)")
    args = ap.parse_args()

    import gguf
    from gguf import GGMLQuantizationType as T
    from gguf import quants

    import oracle  # only for the ref-kernel loader and the Q4_K packer that produces *input* bytes

    # 1. I2_S fixtures --------------------------------------------------------------------------------------------
    fx = os.path.join(args.reference, "tests", "fixtures")
    manifest = json.load(open(os.path.join(fx, "fixture_manifest.json")))["fixtures"]
    sha = {}
    for name in ("fixture_i2s_upstream.bin", "expected_i2s_upstream_f32.bin", "gguf_slice_blk0_v.bin"):
        shutil.copyfile(os.path.join(fx, name), os.path.join(HERE, name))
        digest = hashlib.sha256(open(os.path.join(HERE, name), "rb").read()).hexdigest()
        want = manifest[name].get("packed_fixture_sha256") or manifest[name].get("expected_f32_sha256")
        assert digest == want, (name, digest, want)
        sha[name] = digest
    meta = {
        "sha256": sha,
        "fixture_i2s_upstream_scale": 1.625,
        "gguf_slice_scale": 2.2931101322,
        "gguf_slice_counts_neg_zero_pos": [48, 38, 42],
        "upstream_counts_neg_zero_pos": [86, 85, 85],
        "gguf_py_version": getattr(gguf, "__version__", "0.19.0"),
    }

    # 2. gguf-py vectors ------------------------------------------------------------------------------------------
    rng = np.random.default_rng(20261125)
    x = rng.standard_normal((12, 512)).astype(np.float32)
    x[1] *= 0.02
    x[2] = 0.0
    x[3, :32] = 0.0                        # an all-zero block inside a non-zero row
    x[4] *= 1e-6                           # fp16-subnormal scales
    x[5, :32] = (np.arange(32, dtype=np.float32) - 15.0) * 0.5 + 0.25  # with d = 0.5 below: x/d = k + 0.5, all ties
    x[5, 0] = -127.0 / 2                   # amax 63.5 -> d = 0.5 exactly
    x[6] *= 300.0
    np.savez_compressed(
        os.path.join(HERE, "gguf_q8_0_q4_0.npz"),
        x=x,
        q8_0=quants.quantize(x, T.Q8_0),
        q4_0=quants.quantize(x, T.Q4_0),
        deq_q8_0=quants.dequantize(quants.quantize(x, T.Q8_0), T.Q8_0),
        deq_q4_0=quants.dequantize(quants.quantize(x, T.Q4_0), T.Q4_0),
    )

    # Q4_K: block bytes are inputs; take packer output plus fully random payloads with hand-set fp16 fields.
    wk = (rng.standard_normal((6, 1024)) * 0.02).astype(np.float32)
    q4k = oracle.quantize_q4_K(wk)
    rnd = rng.integers(0, 256, size=(4, 4 * 144), dtype=np.uint8)
    for r in range(4):
        for b in range(4):
            d = np.float16([0.01, 1.0, 6.1e-5 / 4, 0.0][r])       # incl. an fp16 subnormal and zero
            dmin = np.float16([0.02, 0.5, 1e-3, 0.25][b])
            rnd[r, b * 144:b * 144 + 2] = np.frombuffer(d.tobytes(), np.uint8)
            rnd[r, b * 144 + 2:b * 144 + 4] = np.frombuffer(dmin.tobytes(), np.uint8)
    rnd[0, 4:16] = 0xFF                    # every 6-bit scale and min at 63
    q4k_all = np.concatenate([q4k.reshape(-1), rnd.reshape(-1)])
    np.savez_compressed(os.path.join(HERE, "gguf_q4_K.npz"), q4_K=q4k_all,
                        deq=quants.dequantize(q4k_all.reshape(1, -1), T.Q4_K).reshape(-1))

    # fp16 conversion table: every fp16 bit pattern widened by numpy, and a sweep of fp32 values narrowed by numpy.
    f = np.concatenate([rng.standard_normal(4096).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 1e3, 7e4)])
    f = np.concatenate([f, np.float32([0.0, -0.0, 65504.0, 65520.0, 65519.99, 5.96e-8, 2.98e-8, 2.9802322e-8,
                                       np.inf, -np.inf])])
    np.savez_compressed(os.path.join(HERE, "fp16.npz"), f32=f, f16=f.astype(np.float16).view(np.uint16))

    # 3. the reference's I2_S CPU kernel on seeded inputs ----------------------------------------------------------
    assert oracle.ref_available(), "build oracle/_ref first: make -C oracle ref"
    N, K = 40, 640
    packed = rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)   # includes code 3 (+2 in the dot kernel)
    act = rng.integers(-127, 128, size=(3, K), dtype=np.int8)
    out = np.stack([oracle.ref_vec_dot_i2_i8_s(packed, act[m], N, K) for m in range(3)])
    np.savez_compressed(os.path.join(HERE, "i2s_ref_kernel.npz"), packed=packed, act=act, out=out)

    json.dump(meta, open(os.path.join(HERE, "golden_meta.json"), "w"), indent=1, sort_keys=True)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
