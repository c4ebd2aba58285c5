"""Regenerate the committed fixtures of this directory.

  python tests/golden/make_golden.py [path-to-reference-checkout]

1. ``reference_hashes.json`` -- the sha256 values the reference itself commits for this
   path, read verbatim from ``tests/cross_substrate_identity/<workload>/reference_hashes.toml``
   (with the workload's shape and seed from ``manifest.toml``).  These pin the oracle.
2. ``oracle_hashes.json`` -- sha256 values produced by the (pinned) CPU oracle for shapes
   the reference commits no hash for: the benchmark configurations and an overflow case
   that tells wrap from saturate.  They are SELF-GENERATED; the rule behind them is pinned
   by the reference's own hashes above.
"""
from __future__ import annotations

import json
import os
import sys
import tomllib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle as O  # noqa: E402

WORKLOADS = [
    "gemm-i8-64x64x64", "gemm-i8-mt-64x64x64", "gemm-i8-vnni-64x64x64",
    "gemm-q16-64x64x64", "gemm-q16-fused-64x64x64",
    "gemv-q16-256x256", "gemv-i16-256x256",
    "dot-l2-q16", "dot-l1-q16", "dot-i16-4096",
]


def from_reference(ref: str) -> dict:
    out = {}
    base = os.path.join(ref, "tests", "cross_substrate_identity")
    for w in WORKLOADS:
        with open(os.path.join(base, w, "reference_hashes.toml"), "rb") as f:
            hashes = tomllib.load(f)
        with open(os.path.join(base, w, "manifest.toml"), "rb") as f:
            man = tomllib.load(f)
        out[w] = {
            "source": f"tests/cross_substrate_identity/{w}/reference_hashes.toml",
            "hashes": {k: v for k, v in hashes.items() if isinstance(v, str)},
            "input": man.get("input", {}),
            "symbol": man.get("kernel", {}).get("symbol"),
        }
    return out


def self_generated() -> dict:
    out = {}
    # benchmark configuration 1: int8 256^3, bench seed rule 0xDEADBEEF00000000 ^ n
    seed = 0xDEADBEEF00000000 ^ 256
    g = O.Lcg(seed)
    a, b = g.i8(256 * 256), g.i8(256 * 256)
    out["gemm-i8-256x256x256"] = {"seed": seed, "sha256": O.canonical_hash_i32(O.gemm_i8(a, b, 256, 256, 256))}
    # benchmark configuration 2: Q16.16 1024^3, values in [-4, 4) (shift 13)
    seed = 0xDEADBEEF00000000 ^ 1024
    g = O.Lcg(seed)
    a, b = g.q16(1024 * 1024, 13), g.q16(1024 * 1024, 13)
    c, _ = O.baseline_gemm_q16(a, b, 1024, 1024, 1024)
    band = O.gemm_q16(a[: 8 * 1024], b, 8, 1024, 1024)
    assert np.array_equal(band, c[: 8 * 1024])
    out["gemm-q16-1024x1024x1024-shift13"] = {"seed": seed, "shift": 13, "sha256": O.canonical_hash_i32(c)}
    # int16 GEMM 256^3 (no reference kernel: composed from the int16 row rule); wraps
    seed = 0xDEADBEEF00000000 ^ 256
    g = O.Lcg(seed)
    a, b = g.i16(256 * 256), g.i16(256 * 256)
    out["gemm-i16-256x256x256"] = {"seed": seed, "sha256": O.canonical_hash_i32(O.gemm_i16(a, b, 256, 256, 256))}
    # Q16.16 overflow: full-range i32 operands (shift 0) push sums past 2^31 -> wrap
    seed = 0xDEADBEEF
    g = O.Lcg(seed)
    a, b = g.q16(64 * 64, 0), g.q16(64 * 64, 0)
    c = O.gemm_q16(a, b, 64, 64, 64)
    out["gemm-q16-64x64x64-shift0-wrap"] = {"seed": seed, "shift": 0, "sha256": O.canonical_hash_i32(c)}
    # Q16.16 GEMV 512x130 (K % 8 != 0), the reference bench's anchor shape
    seed = 0xDEADBEEF00000000 ^ ((512 << 20) ^ 130)
    g = O.Lcg(seed)
    w, x = g.q16(512 * 130), g.q16(130)
    out["gemv-q16-512x130"] = {"seed": seed, "sha256": O.canonical_hash_i32(O.gemv_q16(w, x, 512, 130))}
    # the workload set the reference names but has not hashed yet (docs/rfcs/0020-mind-bench-
    # reproducibility-harness.md:93-95: matmul-q16-32 / -256 / -1024, seed 0xDEADBEEF), generated
    # like its committed gemm-q16-fused-64x64x64: A drawn before B, >> 12, B[K][N] used in place
    for n in (32, 256, 1024):
        seed = 0xDEADBEEF
        g = O.Lcg(seed)
        a, b = g.q16(n * n), g.q16(n * n)
        if n <= 256:
            c = O.gemm_q16(a, b, n, n, n)
        else:
            c, _ = O.baseline_gemm_q16(a, b, n, n, n)
            assert np.array_equal(O.gemm_q16(a[: 8 * n], b, 8, n, n), c[: 8 * n])
        out[f"matmul-q16-{n}"] = {"seed": seed, "shift": 12, "sha256": O.canonical_hash_i32(c)}
    return out


def main() -> None:
    # default: a checkout of the reference beside this repository
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.dirname(HERE)), "..", "reference")
    if os.path.isdir(ref):
        with open(os.path.join(HERE, "reference_hashes.json"), "w") as f:
            json.dump(from_reference(ref), f, indent=1, sort_keys=True)
    else:
        print(f"no reference checkout at {ref}: reference_hashes.json left as committed")
    with open(os.path.join(HERE, "oracle_hashes.json"), "w") as f:
        json.dump(self_generated(), f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
