"""The give-up paths of the bounded waits, exercised on a healthy GPU: a barrier at which nothing arrives with a
limit of a fraction of a millisecond.  Nothing here traps, faults or spins without a limit; the launches return
by themselves, the status word names the wait, nothing is stored, and the next normal launch is unaffected."""
import ctypes as C

import numpy as np
import pytest

from hipgpt_b200 import _capi, synth
from oracle import bindings as ob

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
from tests.gpu_util import gpu_mha  # noqa: E402


def _status():
    st = C.c_int(-1)
    _capi.check(_capi.lib().hipgpt_kernel_status(C.byref(st)))
    return st.value


def test_a_wait_that_runs_out_is_reported_and_stores_nothing():
    lib = _capi.lib()
    assert _status() == 0
    canary = torch.full((4096,), -7.0, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _capi.check(lib.hipgpt_debug_wait_expiry(canary.data_ptr(), canary.numel(), 200000, st))     # ~0.1 ms at 1.9 GHz
    torch.cuda.synchronize()
    assert _status() == 907                      # 900 + the site of the wait that ran out; not the one that completed (1),
    assert _status() == 0                        # not the one cut short by the flag (8); read once, then cleared
    assert bool((canary == -7.0).all())          # the block skipped its stores
    # the next normal launch is unaffected
    B, H, S, D = 2, 4, 256, 32
    qkv = synth.qkv_planes(5, B, S, H * D)
    out, _ = gpu_mha(qkv, B, S, H * D, H, True, False)
    assert float(np.abs(out - ob.mha(qkv, B, S, H * D, H, causal=True)[0]).max()) <= 1e-5
    assert _status() == 0
    # limits outside the hook's range are refused
    assert lib.hipgpt_debug_wait_expiry(canary.data_ptr(), canary.numel(), 1 << 30, st) == _capi.ERR_BAD_ARG


def test_a_stalled_grid_barrier_ends_the_persistent_generation_call_with_an_error():
    from hipgpt_b200.generation import GptDecoder, MODE_PERSISTENT
    cfg = dict(V=97, S=48, E=64, L=2, H=2, F=128)
    w = synth.gpt_weights(9, **cfg)
    prompts = synth.token_ids(10, (3, 4), cfg["V"])
    dec = GptDecoder(w, **cfg, max_batch=3)
    want = dec.generate(prompts, 10)[0]                     # graph mode
    dec.set_mode(MODE_PERSISTENT)
    assert np.array_equal(dec.generate(prompts, 10)[0], want)
    _capi.check(_capi.lib().hipgpt_gpt_debug_stall_barrier(dec._h, 400000))      # ~0.2 ms
    with pytest.raises(_capi.HipGPTError, match="grid barrier"):
        dec.generate(prompts, 10)
    assert np.array_equal(dec.generate(prompts, 10)[0], want)                  # the handle stays usable
    dec.close()
