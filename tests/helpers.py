"""Shared fixtures for the tests: seeded synthetic tensors and the reference's
own fixture generator for the K-quant encoder goldens."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "frink_goldens.json")


def goldens():
    with open(GOLDEN) as f:
        t = json.load(f)["tables"]
    return {k: v["values"] for k, v in t.items()}


def xorshift_unit(n, seed):
    """The reference fixtures' generator: 32-bit xorshift, top 24 bits to [-1, 1)
    (crates/frink-quant/src/encode.rs:138-150, encode/testdata.rs:92-100)."""
    out = np.empty(n, np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(s >> 8) / np.float32(8388608.0)) - np.float32(1.0)
    return out


def k_quant_fixture(real_weight_bits):
    """crates/frink-quant/src/encode/testdata.rs:90-135: four shaped synthetic
    super-blocks rounded through f16, then eight real-weight super-blocks given
    as f16 bit patterns."""
    gains = [0.02, 0.05, 0.1, 0.25]
    v = xorshift_unit(4 * 8 * 32, 0xB54CDA26)
    out = np.empty(4 * 256, np.float32)
    for sub in range(32):
        for i in range(32):
            x = np.float32(v[sub * 32 + i])
            if sub == 8:
                s = np.float32(0.0)
            elif sub == 9:
                s = np.float32(0.125)
            elif sub == 10:
                s = np.float32(abs(x) * np.float32(0.05) + np.float32(0.01))
            elif sub == 11:
                s = np.float32(-(np.float32(abs(x) * np.float32(0.05)) + np.float32(0.01)))
            elif sub == 17:
                s = np.float32(x * np.float32(1e-4))
            else:
                s = np.float32(x * np.float32(gains[sub % 4]))
            out[sub * 32 + i] = np.float32(np.float16(s))
    real = np.array(real_weight_bits, np.uint16).view(np.float16).astype(np.float32)
    return np.concatenate([out, real])


def synth_weights(rows, cols, seed):
    """Synthetic weight matrix of the benchmark's distribution, N(0, 0.02^2)."""
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)).astype(np.float32)


def synth_acts(batch, cols, seed):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((batch, cols), dtype=np.float32)


def rel_l2(got, want):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def max_abs_over_inf(got, want):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))
