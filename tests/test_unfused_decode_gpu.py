"""GPU parity tests of the unfused chain and of the split-context decode kernel."""
import numpy as np
import pytest

from hipgpt_b200 import _capi, synth
from oracle import bindings as ob

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
from hipgpt_b200 import launchers  # noqa: E402
from tests.gpu_util import dev  # noqa: E402

GOLDEN = np.load(__import__("os").path.join(__import__("os").path.dirname(__file__), "golden", "attn_golden.npz"))


@pytest.mark.parametrize("shape", [(3, 20, 32), (2, 33, 64), (1, 1, 32), (5, 70, 16), (2, 45, 100), (1, 64, 7)])
def test_unfused_chain(shape):
    Bp, S, D = shape
    Q, K, V = (synth.normal(60 + i, (Bp, S, D)) for i in range(3))
    dQ, dK, dV = dev(Q), dev(K), dev(V)
    d_scores = torch.full((Bp, S, S), float("nan"), device="cuda")
    launchers.launch_scaled_dot_product(dQ, dK, d_scores, Bp, S, D)
    scores = d_scores.cpu().numpy()
    # same summation order, fused multiply-add: equal bit for bit to that arithmetic on the CPU
    assert np.array_equal(scores, ob.sdp(Q, K, Bp, S, D, fma=True))
    np.testing.assert_allclose(scores, ob.sdp(Q, K, Bp, S, D), atol=1e-5, rtol=0)   # the pinned oracle
    d_sm = torch.full((Bp, S, S), float("nan"), device="cuda")
    launchers.launch_softmax(d_scores, d_sm, Bp, S)
    sm = d_sm.cpu().numpy()
    np.testing.assert_allclose(sm, ob.softmax(scores, Bp, S), atol=1e-6, rtol=0)
    d_o = torch.full((Bp, S, D), float("nan"), device="cuda")
    launchers.launch_attention_weighted_sum(d_sm, dV, d_o, Bp, S, D)
    assert np.array_equal(d_o.cpu().numpy(), ob.weighted_sum(sm, V, Bp, S, D, fma=True))
    np.testing.assert_allclose(d_o.cpu().numpy(), ob.weighted_sum(sm, V, Bp, S, D), atol=1e-5, rtol=0)
    # softmax in place, as the reference's signature allows
    launchers.launch_softmax(d_scores, d_scores, Bp, S)
    assert np.array_equal(d_scores.cpu().numpy(), sm)


def test_unfused_chain_takes_more_batch_items_than_one_grid_holds():
    """The reference's kernels index threads by B' * S and take any B'; here the batch index rides on grid.z
    (65535 at most), so larger counts are split over several launches."""
    Bp, S, D = 65535 + 70, 4, 8
    Q, K, V = (synth.normal(80 + i, (Bp, S, D)) for i in range(3))
    dQ, dK, dV = dev(Q), dev(K), dev(V)
    d_scores = torch.full((Bp, S, S), float("nan"), device="cuda")
    d_o = torch.full((Bp, S, D), float("nan"), device="cuda")
    launchers.launch_scaled_dot_product(dQ, dK, d_scores, Bp, S, D)
    launchers.launch_softmax(d_scores, d_scores, Bp, S)
    launchers.launch_attention_weighted_sum(d_scores, dV, d_o, Bp, S, D)
    sm = ob.softmax(ob.sdp(Q, K, Bp, S, D, fma=True), Bp, S)
    got = d_o.cpu().numpy()
    assert np.isfinite(got).all()
    np.testing.assert_allclose(got, ob.weighted_sum(sm, V, Bp, S, D, fma=True), atol=1e-6, rtol=0)


def test_unfused_chain_matches_reference_golden():
    Bp, S, D = (int(x) for x in GOLDEN["trio.shape"])
    dQ, dK, dV = dev(GOLDEN["trio.Q"]), dev(GOLDEN["trio.K"]), dev(GOLDEN["trio.V"])
    d_scores = torch.empty((Bp, S, S), device="cuda")
    d_sm = torch.empty((Bp, S, S), device="cuda")
    d_o = torch.empty((Bp, S, D), device="cuda")
    launchers.launch_scaled_dot_product(dQ, dK, d_scores, Bp, S, D)
    launchers.launch_softmax(d_scores, d_sm, Bp, S)
    launchers.launch_attention_weighted_sum(d_sm, dV, d_o, Bp, S, D)
    np.testing.assert_allclose(d_scores.cpu().numpy(), GOLDEN["trio.scores"], atol=1e-5, rtol=0)
    np.testing.assert_allclose(d_sm.cpu().numpy(), GOLDEN["trio.softmax"], atol=1e-6, rtol=0)
    np.testing.assert_allclose(d_o.cpu().numpy(), GOLDEN["trio.out"], atol=1e-5, rtol=0)


def test_unfused_chain_equals_fused_kernel():
    B, H, S, D = 2, 4, 64, 32
    E = H * D
    qkv = synth.qkv_planes(9, B, S, E)
    from tests.gpu_util import gpu_mha
    fused, fprobs = gpu_mha(qkv, B, S, E, H, False, True)
    q, k, v = (dev(np.ascontiguousarray(qkv[i].reshape(B, S, H, D).transpose(0, 2, 1, 3))) for i in range(3))
    sc = torch.empty((B * H, S, S), device="cuda")
    sm = torch.empty((B * H, S, S), device="cuda")
    o = torch.empty((B * H, S, D), device="cuda")
    launchers.launch_scaled_dot_product(q, k, sc, B * H, S, D)
    launchers.launch_softmax(sc, sm, B * H, S)
    launchers.launch_attention_weighted_sum(sm, v, o, B * H, S, D)
    unf = o.cpu().numpy().reshape(B, H, S, D).transpose(0, 2, 1, 3).reshape(B * S, E)
    np.testing.assert_allclose(unf, fused, atol=1e-5, rtol=0)
    np.testing.assert_allclose(sm.cpu().numpy().reshape(B, H, S, S), fprobs, atol=1e-5, rtol=0)


@pytest.mark.parametrize("shape", [(8, 8, 32, 256, 256), (8, 8, 32, 17, 256), (1, 1, 32, 1, 4), (2, 3, 64, 100, 128),
                                   (3, 2, 128, 77, 80), (2, 2, 16, 50, 64), (1, 2, 48, 33, 40), (2, 1, 200, 70, 70),
                                   (1, 2, 5, 9, 16), (400, 2, 32, 64, 64), (2, 2, 32, 0, 8)])
def test_decode_matches_oracle(shape):
    B, H, D, ctx, cap = shape
    E = H * D
    q = synth.normal(70, (B, E))
    kc = synth.normal(71, (B, cap, E))
    vc = synth.normal(72, (B, cap, E))
    ref = ob.decode_row(q, kc, vc, B, H, D, ctx, cap)
    nbytes = launchers.decode_scratch_bytes(B, H, D, ctx)
    scratch = torch.full((max(nbytes // 4, 1),), float("nan"), device="cuda")
    d_out = torch.full((B, E), float("nan"), device="cuda")
    launchers.mha_decode(dev(q), dev(kc), dev(vc), d_out, scratch if nbytes else None, B, H, D, ctx, cap)
    out = d_out.cpu().numpy()
    assert np.isfinite(out).all()
    assert float(np.max(np.abs(out - ref))) <= 1e-5


def test_decode_rejects_small_scratch():
    B, H, D, ctx = 2, 2, 32, 256
    need = launchers.decode_scratch_bytes(B, H, D, ctx)
    assert need > 0
    z = torch.zeros((B, H * D), device="cuda")
    c = torch.zeros((B, ctx, H * D), device="cuda")
    small = torch.zeros((need // 4 - 1,), device="cuda")
    with pytest.raises(_capi.HipGPTError) as e:
        launchers.mha_decode(z, c, c, z, small, B, H, D, ctx, ctx)
    assert e.value.code == _capi.ERR_SCRATCH


def test_decode_equals_last_row_of_causal_prefill():
    B, H, D, S = 4, 8, 32, 200
    E = H * D
    qkv = synth.qkv_planes(73, B, S, E)
    from tests.gpu_util import gpu_mha
    full, _ = gpu_mha(qkv, B, S, E, H, True, False)
    planes = qkv.reshape(3, B, S, E)
    nbytes = launchers.decode_scratch_bytes(B, H, D, S)
    scratch = torch.empty((max(nbytes // 4, 1),), device="cuda")
    d_out = torch.empty((B, E), device="cuda")
    launchers.mha_decode(dev(planes[0][:, -1]), dev(planes[1]), dev(planes[2]), d_out, scratch, B, H, D, S, S)
    np.testing.assert_allclose(d_out.cpu().numpy(), full.reshape(B, S, E)[:, -1], atol=1e-5, rtol=0)
