"""GPU test of hipgpt_mha_decode_noalloc, the decode entry point for callers that cannot bring
scratch memory: stateless launcher-style code in a per-token loop has no pointer to keep and must
not allocate there, so the partial results of the split-context kernel live in a fixed array
inside the library.  The entry point must give what hipgpt_mha_decode gives with caller scratch,
call after call (the array keeps the previous call's contents), and must refuse what does not fit.

The file name sorts last on purpose: a run that stops at the first failure has then already
run every other test.  The test also passes alone in a fresh process."""
import numpy as np
import pytest

from hipgpt_b200 import _capi, synth
from oracle import bindings as ob

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-5      # the tolerance of the other decode tests


def _call_pair(lib, B, H, D, ctx, cap, seed):
    """(output with caller scratch, output without allocation) for one seeded problem."""
    E = H * D
    q = torch.from_numpy(synth.normal(seed, (B, E))).cuda()
    kc = torch.from_numpy(synth.normal(seed + 1, (B, cap, E))).cuda()
    vc = torch.from_numpy(synth.normal(seed + 2, (B, cap, E))).cuda()
    st = torch.cuda.current_stream().cuda_stream
    nbytes = int(lib.hipgpt_mha_decode_scratch_bytes(B, H, D, ctx))
    scratch = torch.full((max(nbytes // 4, 1),), float("nan"), device="cuda")
    want = torch.full((B, E), float("nan"), device="cuda")
    _capi.check(lib.hipgpt_mha_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), want.data_ptr(),
                                      scratch.data_ptr() if nbytes else None, nbytes, B, H, D, ctx, cap, st))
    got = torch.full((B, E), float("nan"), device="cuda")
    _capi.check(lib.hipgpt_mha_decode_noalloc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), got.data_ptr(),
                                              B, H, D, ctx, cap, st))
    torch.cuda.synchronize()
    # the CPU oracle's single-row attention on the same inputs: the entry point is checked against the
    # reference arithmetic too, not only against its sibling kernel launch
    ref = ob.decode_row(q.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), B, H, D, ctx, cap)
    assert float(np.abs(got.cpu().numpy() - ref).max()) <= TOL
    return want.cpu().numpy(), got.cpu().numpy(), nbytes


def test_two_calls_in_a_row_match_the_caller_scratch_entry_point():
    lib = _capi.lib()
    # first call: 8 prompts x 8 heads over 256 cached positions, several splits -> scratch in use
    want, got, nbytes = _call_pair(lib, 8, 8, 32, 256, 256, seed=500)
    assert nbytes > 0, "this shape must exercise the partial-result array"
    assert np.isfinite(got).all()
    assert float(np.abs(got - want).max()) <= TOL
    # second call, other shape and data, straight after: the array still holds the first call's partials
    want2, got2, nbytes2 = _call_pair(lib, 3, 2, 64, 500, 512, seed=600)
    assert nbytes2 > 0
    assert np.isfinite(got2).all()
    assert float(np.abs(got2 - want2).max()) <= TOL
    # and the first problem again gives the first answer again
    want3, got3, _ = _call_pair(lib, 8, 8, 32, 256, 256, seed=500)
    assert np.array_equal(got3, got) and np.array_equal(want3, want)


def test_requests_beyond_the_fixed_array_are_refused():
    lib = _capi.lib()
    st = torch.cuda.current_stream().cuda_stream
    # 256 rows x 2 splits x 132 floats = 270 KB of partial results: fits
    B, H, D, ctx = 16, 16, 128, 256
    z = torch.zeros((B, H * D), device="cuda")
    c = torch.zeros((B, ctx, H * D), device="cuda")
    assert 0 < int(lib.hipgpt_mha_decode_scratch_bytes(B, H, D, ctx)) <= (1 << 20)
    assert lib.hipgpt_mha_decode_noalloc(z.data_ptr(), c.data_ptr(), c.data_ptr(), z.data_ptr(), B, H, D, ctx, ctx, st) == 0
    # 295 rows x 2 splits x 516 floats = 1.2 MB: does not fit the 1 MiB array
    B, H, D, ctx = 5, 59, 512, 64
    z = torch.zeros((B, H * D), device="cuda")
    c = torch.zeros((B, ctx, H * D), device="cuda")
    assert int(lib.hipgpt_mha_decode_scratch_bytes(B, H, D, ctx)) > (1 << 20)
    rc = lib.hipgpt_mha_decode_noalloc(z.data_ptr(), c.data_ptr(), c.data_ptr(), z.data_ptr(), B, H, D, ctx, ctx, st)
    assert rc == _capi.ERR_SCRATCH
    assert b"use hipgpt_mha_decode" in lib.hipgpt_last_error()
    torch.cuda.synchronize()
