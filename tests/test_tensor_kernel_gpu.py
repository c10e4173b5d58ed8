"""GPU parity tests of the tcgen05 attention kernels (HIPGPT_ALGO_TENSOR) against the
CPU oracle.  The kernels claim fp32-grade results, so they are held to the same tolerance as the
FFMA kernel: max-abs-error <= 1e-5."""
import ctypes as C

import numpy as np
import pytest

from hipgpt_b200 import _capi, synth
from oracle import bindings as ob

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
from tests.gpu_util import gpu_mha  # noqa: E402

TOL = 1e-5


def _status():
    st = C.c_int(-1)
    _capi.check(_capi.lib().hipgpt_kernel_status(C.byref(st)))
    return st.value


# one key tile, tails of the 64-key tile and of the 128-row block, several blocks, both head dims
SHAPES = [(1, 1, 64, 32), (1, 1, 1, 32), (2, 2, 7, 32), (1, 2, 65, 32), (2, 2, 128, 32), (1, 3, 129, 32),
          (2, 2, 200, 32), (2, 8, 256, 32), (1, 1, 513, 32), (1, 2, 64, 64), (2, 2, 130, 64), (1, 2, 300, 64)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
def test_tensor_kernel_matches_oracle(shape, causal):
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(2000 + S + D, B, S, E)
    ref_out, _ = ob.mha(qkv, B, S, E, H, causal=causal)
    out, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR)
    assert _status() == 0
    assert np.isfinite(out).all()
    assert float(np.abs(out - ref_out).max()) <= TOL


# the probabilities come from a second sweep over the key tiles: tails of the tile, of the block and of the
# 4-column store groups (S not a multiple of 4 takes the scalar stores), several tiles per block
PROB_SHAPES = [(1, 1, 1, 32), (2, 2, 7, 32), (1, 2, 64, 32), (1, 2, 65, 32), (2, 2, 128, 32), (1, 3, 129, 32), (2, 2, 200, 32),
               (1, 1, 513, 32), (2, 3, 640, 32), (1, 2, 64, 64), (2, 2, 130, 64), (1, 2, 300, 64), (1, 2, 1024, 64), (32, 8, 256, 32)]


@pytest.mark.parametrize("shape", PROB_SHAPES)
@pytest.mark.parametrize("causal", [False, True])
def test_tensor_kernel_probabilities_match_oracle(shape, causal):
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(2500 + S + D, B, S, E)
    ref_out, ref_probs = ob.mha(qkv, B, S, E, H, causal=causal, want_probs=True)
    out, probs = gpu_mha(qkv, B, S, E, H, causal, True, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_TILED)
    assert _status() == 0
    assert np.isfinite(out).all() and np.isfinite(probs).all()      # the buffers were pre-filled with NaN
    assert float(np.abs(out - ref_out).max()) <= TOL
    assert float(np.abs(probs - ref_probs).max()) <= TOL
    if causal:
        assert np.all(np.triu(probs, 1) == 0.0)
    # the same call without probabilities gives the same output bits: the second sweep only adds stores
    out2, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_TILED)
    assert np.array_equal(out, out2)


@pytest.mark.parametrize("cfg", ["c2", "c3"])
@pytest.mark.parametrize("causal", [False, True])
def test_tensor_kernel_benchmark_shapes(cfg, causal):
    c = synth.CONFIGS[cfg]
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    E = H * D
    qkv = synth.qkv_planes(c["seed"], B, S, E, c["scale"])
    ref_out, _ = ob.mha(qkv, B, S, E, H, causal=causal)
    out, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR)
    assert _status() == 0
    assert float(np.abs(out - ref_out).max()) <= TOL


# the tensor-core kernels one by one, chosen through the `warps` argument of hipgpt_mha_forward_ex
WHOLE_HEAD_SHAPES = [(1, 1, 1, 32), (1, 1, 7, 32), (2, 2, 64, 32), (1, 2, 65, 32), (2, 2, 128, 32), (1, 3, 129, 32),
                     (2, 3, 200, 32), (2, 2, 255, 32), (32, 8, 256, 32), (40, 8, 256, 32), (50, 9, 130, 32), (20, 16, 100, 32)]
KERNEL_SHAPES = ([(_capi.TENSOR_WHOLE_HEAD, s) for s in WHOLE_HEAD_SHAPES] +
                 [(_capi.TENSOR_SPLIT_TF32, s) for s in [(2, 2, 200, 32), (1, 1, 513, 32), (1, 2, 300, 64), (32, 8, 256, 32)]] +
                 [(_capi.TENSOR_TILED, s) for s in [(1, 1, 1, 32), (1, 1, 7, 32), (1, 2, 65, 32), (2, 3, 200, 32), (1, 1, 513, 32),
                                                    (32, 8, 256, 32), (3, 5, 640, 32), (2, 2, 2048, 32), (1, 2, 64, 64),
                                                    (2, 2, 130, 64), (1, 2, 300, 64), (2, 4, 1024, 64), (1, 1, 7, 64)]])


@pytest.mark.parametrize("kernel,shape", KERNEL_SHAPES)
@pytest.mark.parametrize("causal", [False, True])
def test_each_tensor_kernel_matches_oracle(kernel, shape, causal):
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(3000 + S + D, B, S, E)
    ref_out, _ = ob.mha(qkv, B, S, E, H, causal=causal)
    out, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR, warps=kernel)
    assert _status() == 0
    assert np.isfinite(out).all()
    assert float(np.abs(out - ref_out).max()) <= TOL


@pytest.mark.parametrize("shape", [(1, 1, 1, 32), (2, 2, 7, 32), (1, 2, 64, 32), (1, 2, 65, 32), (2, 2, 128, 32), (1, 3, 129, 32), (2, 2, 130, 32),
                                   (2, 3, 200, 32), (2, 2, 255, 32), (32, 8, 256, 32), (41, 8, 256, 32)])
@pytest.mark.parametrize("causal", [False, True])
def test_whole_head_kernel_probabilities_match_oracle(shape, causal):
    """The whole-head kernel reads P back from tensor memory once the row sums are known: no second sweep.  S not a
    multiple of 4 takes the scalar stores; 328 heads make most blocks take three heads in turn."""
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(2700 + S, B, S, E)
    ref_out, ref_probs = ob.mha(qkv, B, S, E, H, causal=causal, want_probs=True)
    out, probs = gpu_mha(qkv, B, S, E, H, causal, True, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_WHOLE_HEAD)
    assert _status() == 0
    assert np.isfinite(out).all() and np.isfinite(probs).all()      # the buffers were pre-filled with NaN
    assert float(np.abs(out - ref_out).max()) <= TOL
    assert float(np.abs(probs - ref_probs).max()) <= TOL
    np.testing.assert_allclose(probs.sum(-1), 1.0, atol=1e-5)
    if causal:
        assert np.all(np.triu(probs, 1) == 0.0)
    out2, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_WHOLE_HEAD)
    assert np.array_equal(out, out2)                                # storing the probabilities changes no output bit


@pytest.mark.parametrize("causal", [False, True])
def test_whole_head_kernel_is_deterministic_and_batch_sliceable(causal):
    """Products are issued in a fixed order, and a block's arithmetic depends on its own (batch, head) only:
    two runs give the same bits, and so does a run on a slice of the batches (what sharding relies on)."""
    B, H, S, D = 6, 40, 256, 32          # 240 heads: most blocks take two
    E = H * D
    qkv = synth.qkv_planes(4242, B, S, E)
    out, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_WHOLE_HEAD)
    out2, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_WHOLE_HEAD)
    assert np.array_equal(out, out2)
    planes = qkv.reshape(3, B, S * E)
    part, _ = gpu_mha(np.ascontiguousarray(planes[:, 2:5]).reshape(-1), 3, S, E, H, causal, False,
                      algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_WHOLE_HEAD)
    assert np.array_equal(part, out.reshape(B, S * E)[2:5].reshape(3 * S, E))
    assert _status() == 0


def test_whole_head_kernel_rescales_values_of_any_magnitude():
    """V is scaled by a power of two per head before it is cut into fp16 parts, so its magnitude does not matter."""
    B, H, S, D = 2, 4, 256, 32
    E = H * D
    for vscale in (1e-30, 1e-6, 1e5, 1e30):
        qkv = synth.qkv_planes(17, B, S, E).reshape(3, B * S, E).copy()
        qkv[2] *= np.float32(vscale)
        ref_out, _ = ob.mha(qkv, B, S, E, H, causal=True)
        out, _ = gpu_mha(qkv, B, S, E, H, True, False, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_WHOLE_HEAD)
        assert _status() == 0
        assert float(np.abs(out - ref_out).max()) <= TOL * vscale * 4       # |V| reaches about 4 vscale


def test_tensor_kernel_refuses_what_it_cannot_do():
    lib = _capi.lib()
    t = torch.zeros((64, 48), device="cuda")
    p = torch.zeros((1, 1, 64, 64), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    # head_dim 48
    assert lib.hipgpt_mha_forward_ex(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None,
                                     1, 64, 48, 1, 0, _capi.ALGO_TENSOR, 0, st) == _capi.ERR_UNSUPPORTED
    # probabilities requested from a kernel that does not store them
    t32 = torch.zeros((64, 32), device="cuda")
    assert lib.hipgpt_mha_forward_ex(t32.data_ptr(), t32.data_ptr(), t32.data_ptr(), t32.data_ptr(), p.data_ptr(),
                                     1, 64, 32, 1, 0, _capi.ALGO_TENSOR, _capi.TENSOR_SPLIT_TF32, st) == _capi.ERR_UNSUPPORTED
    # the whole-head kernel outside its shape: head_dim 64, S > 256
    t64 = torch.zeros((64, 64), device="cuda")
    assert lib.hipgpt_mha_forward_ex(t64.data_ptr(), t64.data_ptr(), t64.data_ptr(), t64.data_ptr(), None,
                                     1, 64, 64, 1, 0, _capi.ALGO_TENSOR, _capi.TENSOR_WHOLE_HEAD, st) == _capi.ERR_UNSUPPORTED
    big = torch.zeros((300, 32), device="cuda")
    assert lib.hipgpt_mha_forward_ex(big.data_ptr(), big.data_ptr(), big.data_ptr(), big.data_ptr(), None,
                                     1, 300, 32, 1, 0, _capi.ALGO_TENSOR, _capi.TENSOR_WHOLE_HEAD, st) == _capi.ERR_UNSUPPORTED
    # an unknown kernel number
    assert lib.hipgpt_mha_forward_ex(t32.data_ptr(), t32.data_ptr(), t32.data_ptr(), t32.data_ptr(), None,
                                     1, 64, 32, 1, 0, _capi.ALGO_TENSOR, 2, st) == _capi.ERR_BAD_ARG


@pytest.mark.parametrize("D", [32, 64])
@pytest.mark.parametrize("want_probs", [False, True])
def test_tiled_kernel_rescales_when_row_maxima_grow(D, want_probs):
    """The tiled kernel keeps the output in tensor memory and moves the reference maximum only when a row's
    maximum grew by more than 2^8; keys whose scores rise steeply along the sequence force that rescale at
    every tile.  The second sweep (probabilities) reuses the final maximum and sum."""
    B, H, S = 1, 2, 640
    E = H * D
    qkv = synth.qkv_planes(78, B, S, E).reshape(3, B * S, E).copy()
    sign = np.sign(qkv[0][:1])
    ramp = (1.0 + np.arange(S, dtype=np.float32) / 40.0)[:, None]
    qkv[1] = sign * ramp * np.float32(np.sqrt(32.0 / D))    # keys grow along the sequence, aligned with every query
    qkv[0] = np.abs(qkv[0]) * sign
    for causal in (False, True):
        ref_out, ref_probs = ob.mha(qkv, B, S, E, H, causal=causal, want_probs=want_probs)
        out, probs = gpu_mha(qkv, B, S, E, H, causal, want_probs, algo=_capi.ALGO_TENSOR, warps=_capi.TENSOR_TILED)
        assert _status() == 0
        assert float(np.abs(out - ref_out).max()) <= 1e-4     # scores reach ~100: the fp32 arithmetic itself is good to ~1e-5 here
        if want_probs:
            assert float(np.abs(probs - ref_probs).max()) <= 1e-4


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("want_probs", [False, True])
def test_tiled_kernel_in_several_groups_of_batches(monkeypatch, causal, want_probs):
    """The tiled kernel cuts a call into groups of batches whose packed K and V stay in L2 (96 MB by default); unmasked
    calls of several groups pack the next group on a second stream.  A 1 MB limit makes a small call take that path:
    7 batches in groups of 1 (unmasked, two buffers in turn) or 2 (causal, a ragged last group), three calls in a row."""
    monkeypatch.setenv("HIPGPT_PACK_GROUP_MB", "1")
    B, H, S, D = 7, 2, 512, 64                       # 0.5 MB of packed operands per batch item
    E = H * D
    for rep in range(3):
        qkv = synth.qkv_planes(2900 + rep, B, S, E)
        ref_out, ref_probs = ob.mha(qkv, B, S, E, H, causal=causal, want_probs=want_probs)
        out, probs = gpu_mha(qkv, B, S, E, H, causal, want_probs, algo=_capi.ALGO_TENSOR)
        assert _status() == 0
        assert np.isfinite(out).all()
        assert float(np.abs(out - ref_out).max()) <= TOL
        if want_probs:
            assert float(np.abs(probs - ref_probs).max()) <= TOL
