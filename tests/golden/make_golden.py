"""Writes tests/golden/attn_golden.npz from the REFERENCE's own attention launchers.

Run it where the HipGPT source tree is mounted (oracle/Makefile's REF names the place):

    make -C oracle && python tests/golden/make_golden.py

It calls the reference's launch_multihead_attention / launch_scaled_dot_product /
launch_softmax / launch_attention_weighted_sum (src/hip_kernels.cpp:404-532), compiled for
host cores by oracle/Makefile, on seeded inputs and stores inputs and outputs for small
shapes and digests for larger ones.  The fixture travels to machines without the reference.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from hipgpt_b200 import synth  # noqa: E402
from oracle import bindings as ob  # noqa: E402

# name -> (B, H, S, D, seed, scale); which reference kernel each one reaches
SMALL = {
    "flash_d32": (1, 2, 16, 32, 11, 1.0),      # flash_attention_kernel<32>
    "flash_d64": (2, 2, 9, 64, 12, 1.0),       # flash_attention_kernel<64>
    "fallback_d16": (1, 2, 24, 16, 13, 1.0),   # head_dim not in {32, 64} -> fallback kernel
    "flash_s1": (2, 1, 1, 32, 14, 1.0),        # single key
}
# digests only: (B, H, S, D, seed, scale)
LARGE = {
    "c1": (2, 8, 64, 32, 0, 1.0),              # the smallest benchmark shape
    "fallback_s513": (1, 2, 513, 64, 15, 1.0), # S > 512 -> fallback kernel
    "flash_s512": (1, 1, 512, 32, 16, 0.5),    # largest S the flash kernel takes
}


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    if not ob.have_ref():
        raise SystemExit("oracle/_ref/libhipgpt_ref.so is missing: run `make -C oracle` where the reference is mounted")
    out = {}
    for name, (B, H, S, D, seed, scale) in SMALL.items():
        E = H * D
        qkv = synth.qkv_planes(seed, B, S, E, scale)
        o, p = ob.ref_mha(qkv, B, S, E, H)
        out[f"{name}.shape"] = np.array([B, H, S, D, seed], dtype=np.int64)
        out[f"{name}.qkv"] = qkv
        out[f"{name}.out"] = o
        out[f"{name}.probs"] = p
    for name, (B, H, S, D, seed, scale) in LARGE.items():
        E = H * D
        qkv = synth.qkv_planes(seed, B, S, E, scale)
        o, p = ob.ref_mha(qkv, B, S, E, H)
        out[f"{name}.shape"] = np.array([B, H, S, D, seed], dtype=np.int64)
        out[f"{name}.scale"] = np.array([scale], dtype=np.float64)
        out[f"{name}.qkv_sha256"] = np.array(digest(qkv))
        out[f"{name}.out_sha256"] = np.array(digest(o))
        out[f"{name}.probs_sha256"] = np.array(digest(p))
        out[f"{name}.out_head"] = o.reshape(-1)[:16].copy()
        out[f"{name}.out_rows"] = o[:: max(1, (B * S) // 8)].copy()   # a few whole rows for tolerance checks
    # the unfused trio: [B'][S][D] layout (src/hip_kernels.cpp:455-532)
    Bp, S, D = 3, 20, 32
    Q = synth.normal(21, (Bp, S, D)); K = synth.normal(22, (Bp, S, D)); V = synth.normal(23, (Bp, S, D))
    sc = ob.ref_sdp(Q, K, Bp, S, D)
    sm = ob.ref_softmax(sc, Bp, S)
    ws = ob.ref_weighted_sum(sm, V, Bp, S, D)
    out.update({"trio.shape": np.array([Bp, S, D], dtype=np.int64), "trio.Q": Q, "trio.K": K, "trio.V": V,
                "trio.scores": sc, "trio.softmax": sm, "trio.out": ws})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "attn_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
