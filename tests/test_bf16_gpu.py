"""GPU parity tests of the bf16 tensor-core attention (hipgpt_mha_forward_bf16) against the CPU
oracle.  The oracle computes in fp32 on the same bf16-rounded inputs; the kernel rounds the
probabilities and the output to bf16, so the tolerance is the one stated for a bf16 tensor-core
path: max-abs-error <= 1e-2 on unit-variance data."""
import ctypes as C

import numpy as np
import pytest

from hipgpt_b200 import _capi, launchers, synth
from oracle import bindings as ob

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-2


def _status():
    st = C.c_int(-1)
    _capi.check(_capi.lib().hipgpt_kernel_status(C.byref(st)))
    return st.value


def _run(qkv_f32: np.ndarray, B, S, E, H, causal, variant=0):
    """-> (kernel output as float32 numpy, the bf16-rounded inputs as float32 numpy)"""
    d = torch.from_numpy(qkv_f32.reshape(3, B * S, E)).cuda().bfloat16()
    out = torch.full((B * S, E), float("nan"), dtype=torch.bfloat16, device="cuda")
    launchers.mha_forward_bf16(d, out, B, S, E, H, causal=causal, variant=variant)
    torch.cuda.synchronize()
    return out.float().cpu().numpy(), d.float().cpu().numpy()


# single row, tails of the 128-key tile and of the 256-row block, one and several blocks, long rows
SHAPES = [(1, 1, 1, 64), (2, 2, 7, 64), (1, 2, 64, 64), (1, 1, 128, 64), (1, 3, 129, 64), (2, 2, 256, 64),
          (1, 2, 300, 64), (1, 1, 513, 64), (2, 3, 1024, 64)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("variant", [0, 2])       # the `variant` argument is accepted (0, 1, 2) and ignored
def test_bf16_kernel_matches_oracle(shape, causal, variant):
    B, H, S, D = shape
    E = H * D
    out, rounded = _run(synth.qkv_planes(3000 + S, B, S, E), B, S, E, H, causal, variant)
    ref_out, _ = ob.mha(rounded, B, S, E, H, causal=causal)
    assert _status() == 0
    assert np.isfinite(out).all()
    assert float(np.abs(out - ref_out).max()) <= TOL


def test_bf16_rows_whose_maximum_grows_late():
    """Keys ordered so that every later tile raises the row maxima by far more than the rescale
    threshold: the accumulator in tensor memory has to be rescaled at every tile."""
    B, H, S, D = 1, 2, 640, 64
    E = H * D
    qkv = synth.qkv_planes(77, B, S, E).reshape(3, B * S, E).copy()
    ramp = (1.0 + np.arange(S, dtype=np.float32) / 40.0)[:, None]
    qkv[1] = np.sign(qkv[0][:1]) * ramp          # K rows grow along the sequence, aligned with the first query
    qkv[0] = np.abs(qkv[0]) * np.sign(qkv[0][:1])
    for causal, variant in [(False, 1), (True, 1), (False, 2), (True, 2)]:
        out, rounded = _run(qkv, B, S, E, H, causal, variant)
        ref_out, _ = ob.mha(rounded, B, S, E, H, causal=causal)
        assert _status() == 0
        assert float(np.abs(out - ref_out).max()) <= TOL


def test_bf16_scaling_config_sample():
    """The scaling config's shape (S=2048, head_dim 64) on a slice of its batch; the first row of a
    causal head must reproduce its value row exactly (one probability of 1)."""
    c = synth.CONFIGS["c5"]
    B, H, S, D = 2, c["H"], c["S"], c["D"]
    E = H * D
    out, rounded = _run(synth.qkv_planes(c["seed"], B, S, E, c["scale"]), B, S, E, H, True)
    assert _status() == 0
    v = rounded.reshape(3, B, S, E)[2]
    assert np.array_equal(out.reshape(B, S, E)[:, 0], v[:, 0])
    ref_out, _ = ob.mha(rounded, B, S, E, H, causal=True)
    assert float(np.abs(out - ref_out).max()) <= TOL


def test_bf16_rejects_other_head_dims_and_bad_configs():
    lib = _capi.lib()
    x = torch.zeros(3 * 64 * 96, dtype=torch.bfloat16, device="cuda")
    o = torch.zeros(64 * 96, dtype=torch.bfloat16, device="cuda")
    assert lib.hipgpt_mha_forward_bf16(x.data_ptr(), x.data_ptr(), x.data_ptr(), o.data_ptr(), 1, 64, 96, 3, 0, None) == _capi.ERR_UNSUPPORTED   # head_dim 32
    assert lib.hipgpt_mha_forward_bf16(x.data_ptr(), x.data_ptr(), x.data_ptr(), o.data_ptr(), 1, 64, 96, 0, 0, None) == _capi.ERR_BAD_ARG
    assert lib.hipgpt_mha_forward_bf16(x.data_ptr(), x.data_ptr(), x.data_ptr(), o.data_ptr(), 1, 64, 96, 5, 0, None) == _capi.ERR_BAD_ARG
    assert lib.hipgpt_mha_forward_bf16(None, x.data_ptr(), x.data_ptr(), o.data_ptr(), 1, 64, 64, 1, 0, None) == _capi.ERR_NULL
    assert lib.hipgpt_mha_forward_bf16(x.data_ptr(), x.data_ptr(), x.data_ptr(), o.data_ptr(), 0, 64, 64, 1, 0, None) == 0      # nothing to do


@pytest.mark.parametrize("shape", [(1, 1, 7, 64), (3, 2, 300, 64), (16, 4, 512, 64)])
@pytest.mark.parametrize("pinned", [False, True])
def test_bf16_host_buffer_call_equals_the_device_call(shape, pinned):
    """hipgpt_mha_forward_bf16_host copies, runs the same kernel on chunks of batches and copies
    back: its output bits are those of the device-pointer call."""
    B, H, S, D = shape
    E = H * D
    h_qkv = torch.from_numpy(synth.qkv_planes(4000 + S, B, S, E).reshape(3, B * S, E)).bfloat16()
    h_out = torch.full((B * S, E), float("nan"), dtype=torch.bfloat16)
    if pinned:
        h_qkv, h_out = h_qkv.pin_memory(), h_out.pin_memory()
    for causal in (False, True):
        launchers.mha_forward_bf16_host(h_qkv, h_out, B, S, E, H, causal=causal)
        d_out = torch.empty((B * S, E), dtype=torch.bfloat16, device="cuda")
        launchers.mha_forward_bf16(h_qkv.cuda(), d_out, B, S, E, H, causal=causal)
        torch.cuda.synchronize()
        assert _status() == 0
        assert torch.equal(h_out, d_out.cpu())
    _capi.lib().hipgpt_release_workspace()
    # head_dim other than 64 is refused
    bad = torch.zeros((3, 64, 96), dtype=torch.bfloat16)
    assert _capi.lib().hipgpt_mha_forward_bf16_host(bad.data_ptr(), bad.data_ptr(), 1, 64, 96, 3, 0) == _capi.ERR_UNSUPPORTED
