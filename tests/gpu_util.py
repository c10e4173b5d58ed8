"""Helpers of the GPU parity tests: device buffers through torch, calls through the C ABI."""
import numpy as np
import torch

from hipgpt_b200 import _capi


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def gpu_mha(qkv: np.ndarray, B, S, E, H, causal=False, want_probs=False, algo=_capi.ALGO_AUTO, warps=0, fill=None):
    """hipgpt_mha_forward_ex on device copies of three stacked planes -> (out, probs|None) as numpy.
    Output buffers are pre-filled with NaN so that anything the kernel does not write shows."""
    lib = _capi.lib()
    d_qkv = dev(qkv.reshape(3, B * S, E))
    d_out = torch.full((B * S, E), float("nan") if fill is None else fill, dtype=torch.float32, device="cuda")
    d_probs = torch.full((B, H, S, S), float("nan"), dtype=torch.float32, device="cuda") if want_probs else None
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.hipgpt_mha_forward_ex(d_qkv[0].data_ptr(), d_qkv[1].data_ptr(), d_qkv[2].data_ptr(), d_out.data_ptr(),
                                   d_probs.data_ptr() if want_probs else None, B, S, E, H, int(causal), algo, warps, st)
    _capi.check(rc)
    torch.cuda.synchronize()
    return d_out.cpu().numpy(), (d_probs.cpu().numpy() if want_probs else None)
