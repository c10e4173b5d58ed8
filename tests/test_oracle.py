"""CPU tests of the oracle: against the committed golden vectors (outputs of the reference's
own launchers, see tests/golden/make_golden.py), against the reference build where the
HipGPT tree is mounted, and against independent float64 numpy arithmetic."""
import hashlib
import os

import numpy as np
import pytest

from hipgpt_b200 import synth
from oracle import bindings as ob

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "attn_golden.npz"))
SMALL = ["flash_d32", "flash_d64", "fallback_d16", "flash_s1"]
LARGE = ["c1", "fallback_s513", "flash_s512"]


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _np_attention(qkv, B, S, E, H, causal):
    """float64 softmax(QK^T/sqrt(D))V, no shortcuts."""
    D = E // H
    q, k, v = (qkv[i].astype(np.float64).reshape(B, S, H, D).transpose(0, 2, 1, 3) for i in range(3))
    s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(D)
    if causal:
        s = np.where(np.tril(np.ones((S, S), dtype=bool)), s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    o = (p @ v).transpose(0, 2, 1, 3).reshape(B * S, E)
    return o, p


@pytest.mark.parametrize("name", SMALL)
def test_oracle_equals_golden_small_bitwise(name):
    B, H, S, D, _ = (int(x) for x in GOLDEN[f"{name}.shape"])
    E = H * D
    out, probs = ob.mha(GOLDEN[f"{name}.qkv"], B, S, E, H, causal=False, want_probs=True)
    assert np.array_equal(out, GOLDEN[f"{name}.out"])
    assert np.array_equal(probs, GOLDEN[f"{name}.probs"])


@pytest.mark.parametrize("name", LARGE)
def test_oracle_equals_golden_digest(name):
    B, H, S, D, seed = (int(x) for x in GOLDEN[f"{name}.shape"])
    E = H * D
    qkv = synth.qkv_planes(seed, B, S, E, float(GOLDEN[f"{name}.scale"][0]))
    out, probs = ob.mha(qkv, B, S, E, H, causal=False, want_probs=True)
    rows = out[:: max(1, (B * S) // 8)]
    # tolerance check first: it holds even if this machine's libm rounds an input differently
    np.testing.assert_allclose(rows, GOLDEN[f"{name}.out_rows"], atol=1e-6, rtol=0)
    if _sha(qkv) != str(GOLDEN[f"{name}.qkv_sha256"]):
        pytest.skip("seeded inputs differ in the last bit on this machine (libm); digest not comparable")
    assert _sha(out) == str(GOLDEN[f"{name}.out_sha256"])
    assert _sha(probs) == str(GOLDEN[f"{name}.probs_sha256"])


def test_trio_equals_golden_bitwise():
    Bp, S, D = (int(x) for x in GOLDEN["trio.shape"])
    sc = ob.sdp(GOLDEN["trio.Q"], GOLDEN["trio.K"], Bp, S, D)
    assert np.array_equal(sc, GOLDEN["trio.scores"])
    sm = ob.softmax(sc, Bp, S)
    assert np.array_equal(sm, GOLDEN["trio.softmax"])
    ws = ob.weighted_sum(sm, GOLDEN["trio.V"], Bp, S, D)
    assert np.array_equal(ws, GOLDEN["trio.out"])


@pytest.mark.skipif(not ob.have_ref(), reason="reference build absent (HipGPT tree not mounted here)")
@pytest.mark.parametrize("shape", [(2, 8, 64, 32), (1, 3, 33, 64), (2, 2, 17, 16), (1, 2, 513, 32),
                                   (1, 1, 600, 64), (1, 4, 5, 48), (3, 1, 1, 32)])
def test_oracle_equals_reference_build_bitwise(shape):
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(100 + S, B, S, E)
    out, probs = ob.mha(qkv, B, S, E, H, causal=False, want_probs=True)
    rout, rprobs = ob.ref_mha(qkv, B, S, E, H)
    assert np.array_equal(out, rout)
    assert np.array_equal(probs, rprobs)
    # skipping the block rows that repeat the same query changes nothing
    uout, uprobs = ob.ref_mha(qkv, B, S, E, H, unique_rows_only=True)
    assert np.array_equal(uout, rout) and np.array_equal(uprobs, rprobs)


@pytest.mark.skipif(not ob.have_ref(), reason="reference build absent (HipGPT tree not mounted here)")
def test_trio_equals_reference_build_bitwise():
    Bp, S, D = 4, 37, 64
    Q, K, V = (synth.normal(30 + i, (Bp, S, D)) for i in range(3))
    sc = ob.sdp(Q, K, Bp, S, D)
    assert np.array_equal(sc, ob.ref_sdp(Q, K, Bp, S, D))
    sm = ob.softmax(sc, Bp, S)
    assert np.array_equal(sm, ob.ref_softmax(sc, Bp, S))
    assert np.array_equal(ob.weighted_sum(sm, V, Bp, S, D), ob.ref_weighted_sum(sm, V, Bp, S, D))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("path", ["flash", "fallback"])
def test_oracle_against_float64(causal, path):
    B, H, S, D = 2, 3, 50, 32
    E = H * D
    qkv = synth.qkv_planes(5, B, S, E)
    out, probs = ob.mha(qkv, B, S, E, H, causal=causal, want_probs=True, path=path)
    o64, p64 = _np_attention(qkv, B, S, E, H, causal)
    np.testing.assert_allclose(out, o64, atol=2e-6, rtol=0)
    np.testing.assert_allclose(probs, p64, atol=1e-6, rtol=0)
    np.testing.assert_allclose(probs.sum(-1), 1.0, atol=1e-5)
    if causal:
        assert np.all(np.triu(probs, 1) == 0.0)   # exactly zero above the diagonal


def test_flash_and_fallback_and_trio_agree():
    B, H, S, D = 2, 2, 40, 32
    E = H * D
    qkv = synth.qkv_planes(9, B, S, E)
    a, _ = ob.mha(qkv, B, S, E, H, path="flash")
    b, _ = ob.mha(qkv, B, S, E, H, path="fallback")
    np.testing.assert_allclose(a, b, atol=1e-6, rtol=0)
    # trio on head-contiguous copies
    q, k, v = (np.ascontiguousarray(qkv[i].reshape(B, S, H, D).transpose(0, 2, 1, 3)).reshape(B * H, S, D)
               for i in range(3))
    sm = ob.softmax(ob.sdp(q, k, B * H, S, D), B * H, S)
    o = ob.weighted_sum(sm, v, B * H, S, D).reshape(B, H, S, D).transpose(0, 2, 1, 3).reshape(B * S, E)
    np.testing.assert_allclose(a, o, atol=1e-6, rtol=0)


def test_dispatch_rule_follows_launcher():
    lib = ob.oracle_lib()
    for (S, D, want) in [(64, 32, 1), (512, 64, 1), (513, 64, 2), (64, 16, 2), (8, 128, 2)]:
        B, H = 1, 1
        qkv = synth.qkv_planes(1, B, S, D)
        out = np.zeros((S, D), dtype=np.float32)
        rc = lib.oracle_mha_dispatch(ob._f(qkv), ob._f(out), None, B, S, D, H, 0)
        assert rc == want
    assert lib.oracle_mha_dispatch(None, None, None, 1, 4, 30, 4, 0) == -1   # E % H != 0
    assert lib.oracle_mha_dispatch(None, None, None, 1, 4, 32, 0, 0) == -1   # H <= 0


def test_decode_row_matches_last_row_of_causal_prefill():
    B, H, D, S = 3, 4, 32, 29
    E = H * D
    qkv = synth.qkv_planes(17, B, S, E)
    full, _ = ob.mha(qkv, B, S, E, H, causal=True, path="flash")
    q_last = np.ascontiguousarray(qkv[0].reshape(B, S, E)[:, -1])
    kc = np.ascontiguousarray(qkv[1].reshape(B, S, E))
    vc = np.ascontiguousarray(qkv[2].reshape(B, S, E))
    row = ob.decode_row(q_last, kc, vc, B, H, D, ctx=S, cap=S)
    assert np.array_equal(row, full.reshape(B, S, E)[:, -1])


def test_empty_inputs():
    out, probs = ob.mha(np.zeros((3, 0, 32), dtype=np.float32), 0, 4, 32, 1, want_probs=True)
    assert out.shape == (0, 32) and probs.shape == (0, 1, 4, 4)
    out, _ = ob.mha(np.zeros((3, 0, 32), dtype=np.float32), 2, 0, 32, 1)
    assert out.shape == (0, 32)


def test_synth_is_deterministic_and_normal():
    a = synth.normal(3, (1000, 64))
    b = synth.normal(3, (1000, 64))
    assert np.array_equal(a, b)
    assert abs(float(a.mean())) < 0.02 and abs(float(a.std()) - 1.0) < 0.02
    assert not np.array_equal(a, synth.normal(4, (1000, 64)))
    ids = synth.token_ids(3, (8, 16), 5000)
    assert ids.min() >= 0 and ids.max() < 5000


# ---- the pieces around the attention call in the reference's generation loop ------------------------
needs_ref = pytest.mark.skipif(not ob.have_ref(), reason="reference build absent (HipGPT tree not mounted here)")


@needs_ref
def test_oracle_dropout_equals_reference_build_bitwise():
    """The oracle's restatement of launch_dropout_forward (src/hip_kernels.cpp:944-970, generator :24-42)
    against the reference's own code built for the host, at the element counts of the generation window
    (256 x 256), of a longer window and of the training batch."""
    rng = np.random.default_rng(5)
    for n_rows, E in [(256, 256), (1024, 256), (8192, 256)]:
        x = rng.standard_normal(n_rows * E).astype(np.float32)
        ref_out, ref_mask = ob.ref_dropout_forward(x, 0.1, n_rows, E)
        assert np.array_equal(ob.dropout_oracle(x, 0.1), ref_out)
        if n_rows * E <= 185384:
            # the generator's first draw is tiny for small element indices: everything is dropped
            assert not ref_mask.any()
        else:
            assert ref_mask.any()


@needs_ref
def test_reference_embedding_matches_the_oracle_arithmetic():
    """tok[id] + pos[t], and a zero row for an id outside the vocabulary (src/hip_kernels.cpp:537-581)."""
    rng = np.random.default_rng(6)
    V, S, E = 50, 12, 16
    tok = rng.standard_normal((V, E)).astype(np.float32)
    pos = rng.standard_normal((S, E)).astype(np.float32)
    ids = rng.integers(0, V, size=(2, S)).astype(np.int32)
    ids[0, 3] = -1
    ids[1, 5] = V
    got = ob.ref_embedding_lookup(ids, tok, pos, 2, S, V, E).reshape(2, S, E)
    want = tok[np.clip(ids, 0, V - 1)] + pos[None]
    want[0, 3] = 0
    want[1, 5] = 0
    assert np.array_equal(got, want)


def test_window_generation_oracle_with_reference_dropout_is_the_identity_model():
    """The reference's generation loop (padded window of S ids re-run per token) with its inference-time
    dropout: at 256 x 256 elements the mask is all zeros, every sub-layer output is dropped, and the ids are
    those of (tok[id] + pos[S-1]) Wout.  Without dropout the layers matter and the ids differ."""
    g = synth.GPT_DEFAULT
    V, S, E, L, H, F = g["V"], g["S"], g["E"], g["L"], g["H"], g["F"]
    w = synth.gpt_weights(3, **g)
    prompts = synth.token_ids(3, (2, 16), V, stream=1)
    ids, _ = ob.gpt_generate_window(w, V, S, E, L, H, F, prompts, 2, 0.1)
    tok = w[:V * E].reshape(V, E)
    pos = w[V * E:V * E + S * E].reshape(S, E)
    wout = w[-E * V:].reshape(E, V)
    first = ((tok[prompts[:, -1]] + pos[S - 1]).astype(np.float64) @ wout.astype(np.float64)).argmax(1)
    assert ids[:, 0].tolist() == first.tolist()
    second = ((tok[ids[:, 0]] + pos[S - 1]).astype(np.float64) @ wout.astype(np.float64)).argmax(1)
    assert ids[:, 1].tolist() == second.tolist()
    ids0, _ = ob.gpt_generate_window(w, V, S, E, L, H, F, prompts, 2, 0.0)
    assert ids0.tolist() != ids.tolist()
