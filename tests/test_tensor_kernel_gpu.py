"""GPU parity tests of the tcgen05 split-TF32 attention kernel (HIPGPT_ALGO_TENSOR) against the
CPU oracle.  The kernel claims fp32-grade results, so it is held to the same tolerance as the
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
    out, probs = gpu_mha(qkv, B, S, E, H, causal, True, algo=_capi.ALGO_TENSOR)
    assert _status() == 0
    assert np.isfinite(out).all() and np.isfinite(probs).all()      # the buffers were pre-filled with NaN
    assert float(np.abs(out - ref_out).max()) <= TOL
    assert float(np.abs(probs - ref_probs).max()) <= TOL
    if causal:
        assert np.all(np.triu(probs, 1) == 0.0)
    # the same call without probabilities gives the same output bits: the second sweep only adds stores
    out2, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR)
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


# tile variants of the kernel, chosen through the `warps` argument of hipgpt_mha_forward_ex:
# 2 = 128-key tiles with two workers per row (head_dim 32), 3 = persistent blocks over a tile stream
@pytest.mark.parametrize("variant,shape", [(2, (2, 2, 200, 32)), (2, (4, 8, 256, 32)), (2, (1, 1, 513, 32)),
                                           (3, (2, 2, 200, 32)), (3, (32, 8, 256, 32)), (3, (1, 2, 300, 64)),
                                           (3, (3, 40, 130, 32)), (3, (2, 4, 1024, 64)),
                                           # 4 = two query tiles per block with the output accumulated in tensor memory,
                                           # 5 = TF32 main products + FP16 correction products (both head_dim 32)
                                           (4, (1, 1, 7, 32)), (4, (2, 3, 200, 32)), (4, (1, 1, 513, 32)), (4, (32, 8, 256, 32)),
                                           (4, (2, 2, 2048, 32)),
                                           (5, (1, 1, 1, 32)), (5, (1, 1, 7, 32)), (5, (1, 2, 65, 32)), (5, (2, 3, 200, 32)),
                                           (5, (1, 1, 513, 32)), (5, (32, 8, 256, 32)), (5, (3, 5, 640, 32)), (5, (2, 2, 2048, 32)),
                                           (5, (1, 2, 64, 64)), (5, (2, 2, 130, 64)), (5, (1, 2, 300, 64)), (5, (2, 4, 1024, 64)),
                                           (5, (1, 1, 7, 64))])
@pytest.mark.parametrize("causal", [False, True])
def test_tensor_kernel_variants_match_oracle(variant, shape, causal):
    B, H, S, D = shape
    E = H * D
    qkv = synth.qkv_planes(3000 + S + D, B, S, E)
    ref_out, _ = ob.mha(qkv, B, S, E, H, causal=causal)
    out, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR, warps=variant)
    assert _status() == 0
    assert np.isfinite(out).all()
    assert float(np.abs(out - ref_out).max()) <= TOL


def test_tensor_kernel_refuses_what_it_cannot_do():
    lib = _capi.lib()
    t = torch.zeros((64, 48), device="cuda")
    p = torch.zeros((1, 1, 64, 64), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    # head_dim 48
    assert lib.hipgpt_mha_forward_ex(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None,
                                     1, 64, 48, 1, 0, _capi.ALGO_TENSOR, 0, st) == _capi.ERR_UNSUPPORTED
    # probabilities requested from a variant that does not store them (only the default one does)
    t32 = torch.zeros((64, 32), device="cuda")
    for variant in (1, 2, 3, 4):
        assert lib.hipgpt_mha_forward_ex(t32.data_ptr(), t32.data_ptr(), t32.data_ptr(), t32.data_ptr(), p.data_ptr(),
                                         1, 64, 32, 1, 0, _capi.ALGO_TENSOR, variant, st) == _capi.ERR_UNSUPPORTED


@pytest.mark.parametrize("variant", [4, 5])
def test_accumulating_variants_rescale_when_row_maxima_grow(variant):
    """Variants that keep the output in tensor memory move the reference maximum only when a row's
    maximum grew by more than 2^8; keys whose scores rise steeply along the sequence force that
    rescale at every tile."""
    B, H, S, D = 1, 2, 640, 32
    E = H * D
    qkv = synth.qkv_planes(78, B, S, E).reshape(3, B * S, E).copy()
    sign = np.sign(qkv[0][:1])
    ramp = (1.0 + np.arange(S, dtype=np.float32) / 40.0)[:, None]
    qkv[1] = sign * ramp                      # keys grow along the sequence, aligned with every query
    qkv[0] = np.abs(qkv[0]) * sign
    for causal in (False, True):
        ref_out, _ = ob.mha(qkv, B, S, E, H, causal=causal)
        out, _ = gpu_mha(qkv, B, S, E, H, causal, False, algo=_capi.ALGO_TENSOR, warps=variant)
        assert _status() == 0
        assert float(np.abs(out - ref_out).max()) <= 1e-4     # scores reach ~100: the fp32 arithmetic itself is good to ~1e-5 here


@pytest.mark.parametrize("variant", [4])
def test_head_dim_32_variants_refuse_other_head_dims(variant):
    lib = _capi.lib()
    t = torch.zeros((64, 64), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert lib.hipgpt_mha_forward_ex(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None,
                                     1, 64, 64, 1, 0, _capi.ALGO_TENSOR, variant, st) == _capi.ERR_UNSUPPORTED
