"""Greedy KV-cache generation: the CPU oracle against plain numpy on a tiny model (CPU), and the
GPU driver against the oracle: token ids must be identical, logits within 1e-4."""
import numpy as np
import pytest

from hipgpt_b200 import synth
from oracle import bindings as ob


def _numpy_generate(w, V, S, E, L, H, F, prompts, n_new, margins=None):
    """Independent float64 restatement: full causal recompute per step, no cache."""
    D = E // H
    off = 0

    def take(*shape):
        nonlocal off
        n = int(np.prod(shape))
        a = w[off:off + n].astype(np.float64).reshape(shape)
        off += n
        return a
    tok, pos = take(V, E), take(S, E)
    layers = []
    for _ in range(L):
        layers.append(dict(wqkv=take(E, 3 * E), wo=take(E, E), w1=take(E, F), w2=take(F, E), bqkv=take(3 * E), bo=take(E),
                           b1=take(F), b2=take(E), g1=take(E), be1=take(E), g2=take(E), be2=take(E)))
    wout = take(E, V)

    def ln(x, g, b):
        m = x.mean(-1, keepdims=True)
        v = ((x - m) ** 2).mean(-1, keepdims=True)
        return g * (x - m) / np.sqrt(v + 1e-5) + b
    out = np.zeros((prompts.shape[0], n_new), dtype=np.int64)
    for bi, prm in enumerate(prompts):
        seq = list(prm)
        for i in range(n_new):
            T = len(seq)
            x = tok[seq] + pos[:T]
            for lw in layers:
                h = ln(x, lw["g1"], lw["be1"])
                qkv = h @ lw["wqkv"] + lw["bqkv"]
                q, k, v = (qkv[:, j * E:(j + 1) * E].reshape(T, H, D).transpose(1, 0, 2) for j in range(3))
                s = q @ k.transpose(0, 2, 1) / np.sqrt(D)
                s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
                p = np.exp(s - s.max(-1, keepdims=True))
                p /= p.sum(-1, keepdims=True)
                a = (p @ v).transpose(1, 0, 2).reshape(T, E)
                x = x + a @ lw["wo"] + lw["bo"]
                h = ln(x, lw["g2"], lw["be2"])
                x = x + np.maximum(h @ lw["w1"] + lw["b1"], 0) @ lw["w2"] + lw["b2"]
            logits = x[-1] @ wout
            nxt = int(np.argmax(logits))
            out[bi, i] = nxt
            if margins is not None:
                top2 = np.partition(logits, -2)[-2:]
                margins.append(float(top2[1] - top2[0]))
            seq.append(nxt)
    return out


def test_oracle_generation_matches_numpy_on_a_tiny_model():
    cfg = dict(V=50, S=24, E=32, L=2, H=4, F=64)
    w = synth.gpt_weights(9, **cfg, std=0.3)          # wide weights: logits well separated
    assert w.size == ob.gpt_weight_count(**cfg)
    prompts = synth.token_ids(9, (3, 5), cfg["V"])
    for fma in (False, True):
        ids, logits = ob.gpt_generate(w, **cfg, prompts=prompts, n_new=12, fma=fma)
        assert np.array_equal(ids, _numpy_generate(w, **cfg, prompts=prompts, n_new=12))
        assert np.isfinite(logits).all()


def test_oracle_generation_matches_numpy_on_the_default_model():
    """The benchmark's whole generation case (E=256 L=8 H=8 F=1024 V=5000 S=256, weights N(0, 0.02) seed 3, 8 prompts
    of 16 ids, 128 new tokens): all 1024 ids of the fp32 oracle against float64 arithmetic that shares nothing with it,
    with the gap between the two largest logits of every step: the room an fp32 rounding difference (about 1e-6 here)
    has before it changes an id.  Measured: smallest gap 2.9e-5, 4 steps below 1e-4, median 2.4e-2."""
    cfg = dict(synth.GPT_DEFAULT)
    w = synth.gpt_weights(3, **cfg)
    prompts = synth.token_ids(3, (8, 16), cfg["V"])
    n_new = 128
    margins = []
    want = _numpy_generate(w, **cfg, prompts=prompts, n_new=n_new, margins=margins)
    ids, _ = ob.gpt_generate(w, **cfg, prompts=prompts, n_new=n_new, fma=True)
    assert len(margins) == 1024 and min(margins) > 1e-5, f"a step of this seed is decided by {min(margins):.2e}: below fp32 noise"
    assert np.array_equal(ids, want)


def test_oracle_rejects_requests_past_the_position_table():
    cfg = dict(V=50, S=8, E=32, L=1, H=4, F=64)
    w = synth.gpt_weights(1, **cfg)
    with pytest.raises(ValueError):
        ob.gpt_generate(w, **cfg, prompts=np.zeros((1, 5), np.int32), n_new=5)     # 5 + 5 - 1 > 8


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["persistent", "graph"])
@pytest.mark.parametrize("shape", ["tiny", "default"])
def test_gpu_generation_ids_equal_the_oracle(shape, mode):
    pytest.importorskip("torch")
    from hipgpt_b200 import generation
    if shape == "tiny":
        cfg, B, n_prompt, n_new, seed = dict(V=50, S=24, E=32, L=2, H=4, F=64), 3, 5, 12, 9
    else:
        cfg, B, n_prompt, n_new, seed = dict(synth.GPT_DEFAULT), 8, 16, 128, 3      # the benchmark's whole-model case
    w = synth.gpt_weights(seed, **cfg)
    prompts = synth.token_ids(seed, (B, n_prompt), cfg["V"])
    ref_ids, ref_logits = ob.gpt_generate(w, **cfg, prompts=prompts, n_new=n_new, fma=True)
    dec = generation.GptDecoder(w, **cfg, max_batch=B,
                                mode=generation.MODE_PERSISTENT if mode == "persistent" else generation.MODE_GRAPH)
    ids, logits, ms_prompt, ms_decode = dec.generate(prompts, n_new)
    dec.close()
    if not np.array_equal(ids, ref_ids):
        b, i = np.argwhere(ids != ref_ids)[0]
        pytest.fail(f"first differing id at prompt {b}, step {i}: gpu {ids[b, i]} oracle {ref_ids[b, i]}")
    assert float(np.abs(logits - ref_logits).max()) <= 1e-4
    assert ms_prompt > 0 and ms_decode > 0


@pytest.mark.gpu
def test_gpu_generation_forms_agree_and_a_handle_serves_many_requests():
    """The persistent kernel and the replayed graph run the same arithmetic; one handle answers
    requests of different batch sizes and lengths in either form, in any order (the grid barrier's
    generation word and the position word carry over from call to call)."""
    pytest.importorskip("torch")
    from hipgpt_b200 import generation
    cfg = dict(V=300, S=48, E=64, L=3, H=2, F=128)          # head_dim 32
    w = synth.gpt_weights(21, **cfg)
    dec = generation.GptDecoder(w, **cfg, max_batch=5)
    for B, n_prompt, n_new in [(5, 4, 20), (2, 7, 1), (1, 1, 48), (3, 10, 30)]:
        prompts = synth.token_ids(100 + B, (B, n_prompt), cfg["V"])
        ref_ids, ref_logits = ob.gpt_generate(w, **cfg, prompts=prompts, n_new=n_new, fma=True)
        got = {}
        for mode in (generation.MODE_PERSISTENT, generation.MODE_GRAPH, generation.MODE_PERSISTENT):
            dec.set_mode(mode)
            ids, logits, _, _ = dec.generate(prompts, n_new)
            assert np.array_equal(ids, ref_ids)
            assert float(np.abs(logits - ref_logits).max()) <= 1e-4
            got[mode] = logits
        assert float(np.abs(got[generation.MODE_PERSISTENT] - got[generation.MODE_GRAPH]).max()) <= 1e-5
    dec.close()
