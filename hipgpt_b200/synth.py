"""Seeded synthetic inputs for the attention path.

The reference ships no dataset for this path (its only corpus is fetched by
scripts/download_data.sh:16 and is used for training), so every test and benchmark feeds
iid normal activations.  The generator is counter based and depends on nothing but integer
arithmetic and float64 log / sqrt / cos, so the same (seed, shape) gives the same stream on
every machine that the tests, the benchmark and the CPU oracle run on.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    """One splitmix64 finaliser per element of a uint64 array (wrap-around arithmetic)."""
    with np.errstate(over="ignore"):
        z = x + _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform_u64(seed: int, n: int, stream: int = 0) -> np.ndarray:
    """n 64-bit words; element i depends only on (seed, stream, i)."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream)],
                                    dtype=np.uint64))[0]
        idx = np.arange(n, dtype=np.uint64)
        return _splitmix64(base + idx * _GOLDEN)


def normal(seed: int, shape, scale: float = 1.0, stream: int = 0) -> np.ndarray:
    """iid N(0, scale^2) float32 of the given shape: Box-Muller in float64 over pairs of
    53-bit uniforms, rounded once to float32."""
    n = int(np.prod(shape))
    m = (n + 1) // 2
    w = uniform_u64(seed, 2 * m, stream)
    u1 = ((w[0::2] >> np.uint64(11)).astype(np.float64) + 1.0) * (1.0 / 9007199254740992.0)  # (0, 1]
    u2 = (w[1::2] >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)          # [0, 1)
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.empty(2 * m, dtype=np.float64)
    z[0::2] = r * np.cos(2.0 * np.pi * u2)
    z[1::2] = r * np.sin(2.0 * np.pi * u2)
    return (z[:n] * scale).astype(np.float32).reshape(shape)


def token_ids(seed: int, shape, vocab: int, stream: int = 0) -> np.ndarray:
    """Uniform int32 ids in [0, vocab)."""
    n = int(np.prod(shape))
    w = uniform_u64(seed, n, stream)
    return (w % np.uint64(vocab)).astype(np.int32).reshape(shape)


def qkv_planes(seed: int, B: int, S: int, E: int, scale: float = 1.0) -> np.ndarray:
    """The launcher's input: three stacked [B*S, E] planes, Q then K then V
    (src/hip_kernels.cpp:415-417), as one float32 array of shape [3, B*S, E]."""
    return normal(seed, (3, B * S, E), scale)


# The shapes that the benchmark description names: (B, H, S, D, seed, scale).
CONFIGS = {
    "c1": dict(B=2, H=8, S=64, D=32, seed=0, scale=1.0),
    "c2": dict(B=32, H=8, S=256, D=32, seed=1, scale=0.5),
    "c3": dict(B=16, H=8, S=1024, D=64, seed=2, scale=1.0),
    "c5": dict(B=64, H=16, S=2048, D=64, seed=4, scale=1.0),
}


# The whole-model benchmark shape (HipGPT's default hyper-parameters, src/train_gpt.cpp:175-183).
GPT_DEFAULT = dict(V=5000, S=256, E=256, L=8, H=8, F=1024)


def gpt_weights(seed: int, V: int, S: int, E: int, L: int, H: int, F: int, std: float = 0.02) -> np.ndarray:
    """Random-init weight blob in the reference's checkpoint order (src/gpt_model.cpp:355-420,
    src/transformer_layer.cpp:312-405, integer headers left out): matrices N(0, std^2), biases 0,
    layer-norm gamma 1 and beta 0."""
    parts = []
    stream = 0

    def mat(*shape):
        nonlocal stream
        stream += 1
        return normal(seed, shape, std, stream=stream).reshape(-1)

    parts.append(mat(V, E))
    parts.append(mat(S, E))
    for _ in range(L):
        parts += [mat(E, 3 * E), mat(E, E), mat(E, F), mat(F, E)]
        parts += [np.zeros(3 * E, np.float32), np.zeros(E, np.float32), np.zeros(F, np.float32), np.zeros(E, np.float32)]
        parts += [np.ones(E, np.float32), np.zeros(E, np.float32), np.ones(E, np.float32), np.zeros(E, np.float32)]
    parts.append(mat(E, V))
    return np.ascontiguousarray(np.concatenate(parts), dtype=np.float32)


def layer_weights(seed: int, E: int, H: int, F: int, std: float = 0.05) -> np.ndarray:
    """One layer's tensors in checkpoint order (src/transformer_layer.cpp:312-344), every one of them random:
    matrices N(0, std^2), biases N(0, 0.1^2), layer-norm gamma 1 + N(0, 0.1^2), beta N(0, 0.1^2)."""
    del H
    s = [0]

    def rnd(n, scale, shift=0.0):
        s[0] += 1
        return (normal(seed, (n,), scale, stream=s[0]) + np.float32(shift)).astype(np.float32)

    parts = [rnd(E * 3 * E, std), rnd(E * E, std), rnd(E * F, std), rnd(F * E, std),
             rnd(3 * E, 0.1), rnd(E, 0.1), rnd(F, 0.1), rnd(E, 0.1),
             rnd(E, 0.1, 1.0), rnd(E, 0.1), rnd(E, 0.1, 1.0), rnd(E, 0.1)]
    return np.ascontiguousarray(np.concatenate(parts), dtype=np.float32)
