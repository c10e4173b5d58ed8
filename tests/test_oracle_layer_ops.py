"""CPU tests of the oracle's restatements of the launchers either side of attention (projections, layer
norm, embedding, the whole block) and of the attention backward: against independent float64 numpy
arithmetic, and, for the backward, bit for bit against the reference's own source built for the host."""
import numpy as np
import pytest

from hipgpt_b200 import synth
from oracle import bindings as ob


def _np_backward(g, qkv, B, S, E, H, causal):
    D = E // H
    q, k, v = (qkv[i].astype(np.float64).reshape(B, S, H, D).transpose(0, 2, 1, 3) for i in range(3))
    go = g.astype(np.float64).reshape(B, S, H, D).transpose(0, 2, 1, 3)
    s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(D)
    if causal:
        s = np.where(np.tril(np.ones((S, S), dtype=bool)), s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    vd = go @ v.transpose(0, 1, 3, 2)
    w = (p * vd).sum(-1, keepdims=True)
    ds = p * (vd - w)
    dq = ds @ k / np.sqrt(D)
    dk = ds.transpose(0, 1, 3, 2) @ q / np.sqrt(D)
    dv = p.transpose(0, 1, 3, 2) @ go
    return np.stack([x.transpose(0, 2, 1, 3).reshape(B * S, E) for x in (dq, dk, dv)]).reshape(-1)


@pytest.mark.parametrize("shape", [(2, 2, 40, 32), (1, 3, 70, 64), (2, 1, 9, 16)])
@pytest.mark.parametrize("causal", [False, True])
def test_backward_oracle_matches_float64(shape, causal):
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(600 + S, B, S, E)
    g = synth.normal(601 + S, (B * S, E))
    ref = _np_backward(g, qkv.reshape(3, B * S, E), B, S, E, H, causal)
    got = ob.mha_backward(g, qkv, None, B, S, E, H, causal=causal)
    assert float(np.abs(got - ref).max()) <= 2e-6
    # with the stored probabilities of the forward instead of recomputed ones
    _, probs = ob.mha(qkv, B, S, E, H, causal=causal, want_probs=True)
    got2 = ob.mha_backward(g, qkv, probs, B, S, E, H, causal=causal)
    assert float(np.abs(got2 - ref).max()) <= 2e-6


@pytest.mark.skipif(not ob.have_ref(), reason="reference build (oracle/_ref) not present")
@pytest.mark.parametrize("shape", [(2, 2, 40, 32), (1, 2, 300, 64), (1, 3, 33, 16)])
def test_backward_oracle_equals_reference_build_bitwise(shape):
    """The reference's backward kernel has no barriers or shuffles, so the host stand-in runs it; on one
    host thread its atomicAdd order is the oracle's (queries ascending)."""
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(700 + S, B, S, E)
    g = synth.normal(701 + S, (B * S, E))
    _, probs = ob.mha(qkv, B, S, E, H, causal=False, want_probs=True)
    ref = ob.ref_mha_backward(g, qkv, probs, B, S, E, H)
    got = ob.mha_backward(g, qkv, probs, B, S, E, H, causal=False, fma=False)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("M,N,K", [(5, 7, 3), (64, 256, 768), (33, 100, 20)])
def test_matmul_oracle_matches_float64(M, N, K):
    A = synth.normal(11, (M, N))
    W = synth.normal(12, (N, K))
    bias = synth.normal(13, (K,))
    ref = A.astype(np.float64) @ W.astype(np.float64) + bias
    for fma in (False, True):
        got = ob.matmul(A, W, bias, M, N, K, fma=fma)
        assert float(np.abs(got - ref).max()) <= 3e-5 * np.sqrt(N / 100.0)
    assert np.array_equal(ob.matmul(A, W, None, M, N, K), ob.matmul(A, W, np.zeros(K, np.float32), M, N, K))


@pytest.mark.parametrize("E", [256, 64, 100, 1000, 2048])
def test_layer_norm_oracle_orders_agree(E):
    """The library's summation order (32 lanes, butterfly) and the reference kernel's (64-lane waves, tree)
    are rearrangements of the same sums: results agree to rounding, and both match float64."""
    rows = 9
    x = synth.normal(21 + E, (rows, E)) * np.float32(3.0) + np.float32(0.7)
    g = synth.normal(22, (E,))
    b = synth.normal(23, (E,))
    xd = x.astype(np.float64)
    mean = xd.mean(-1, keepdims=True)
    ref = g * (xd - mean) / np.sqrt(((xd - mean) ** 2).mean(-1, keepdims=True) + 1e-5) + b
    a = ob.layer_norm(x, g, b, rows, E, ref_order=False)
    r = ob.layer_norm(x, g, b, rows, E, ref_order=True)
    assert float(np.abs(a - ref).max()) <= 5e-6
    assert float(np.abs(r - ref).max()) <= 5e-6
    assert float(np.abs(a - r).max()) <= 2e-6


@pytest.mark.skipif(not ob.have_ref(), reason="reference build (oracle/_ref) not present")
def test_embedding_oracle_equals_reference_build_bitwise():
    B, S, V, E = 3, 17, 50, 24
    ids = synth.token_ids(5, (B, S), V).copy()
    ids[0, 3] = -1
    ids[2, 5] = V
    tok = synth.normal(31, (V, E))
    pos = synth.normal(32, (S, E))
    assert np.array_equal(ob.embedding(ids, tok, pos, B, S, V, E), ob.ref_embedding_lookup(ids, tok, pos, B, S, V, E))


def test_layer_forward_oracle_matches_float64_without_dropout():
    B, S, E, H, F = 2, 24, 64, 2, 96
    D = E // H
    w = synth.layer_weights(41, E, H, F)
    x = synth.normal(42, (B * S, E))
    got = ob.layer_forward(x, w, B, S, E, H, F, dropout_p=0.0)
    # float64 restatement, including the launcher's reading of the [T][3E] projection as three stacked planes
    o = 0

    def take(n, shape):
        nonlocal o
        a = w[o:o + n].astype(np.float64).reshape(shape)
        o += n
        return a
    wqkv, wo, w1, w2 = take(E * 3 * E, (E, 3 * E)), take(E * E, (E, E)), take(E * F, (E, F)), take(F * E, (F, E))
    bqkv, bo, b1, b2 = take(3 * E, (3 * E,)), take(E, (E,)), take(F, (F,)), take(E, (E,))
    g1, be1, g2, be2 = take(E, (E,)), take(E, (E,)), take(E, (E,)), take(E, (E,))

    def ln(a, g, b):
        m = a.mean(-1, keepdims=True)
        return g * (a - m) / np.sqrt(((a - m) ** 2).mean(-1, keepdims=True) + 1e-5) + b
    xd = x.astype(np.float64)
    qkv = (ln(xd, g1, be1) @ wqkv + bqkv).reshape(-1).reshape(3, B * S, E)       # planes, not columns
    q, k, v = (qkv[i].reshape(B, S, H, D).transpose(0, 2, 1, 3) for i in range(3))
    s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(D)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    att = (p @ v).transpose(0, 2, 1, 3).reshape(B * S, E)
    x1 = xd + att @ wo + bo
    ref = x1 + np.maximum(ln(x1, g2, be2) @ w1 + b1, 0.0) @ w2 + b2
    assert float(np.abs(got - ref).max()) <= 2e-5
